// Cast launcher: every pair over {f16,f32,f64,i8,u8,i16,u16,i32,u32,i64,u64,bool}.
//
// Conversion rules are the reference's (cuda/src/ptx/cast.cu:6-124): static_cast between arithmetic
// types, through float for f16, and `x == 0 ? false : true` into bool.  The reference compiles 100
// of the 144 pairs; the remaining ones (signed<->unsigned integers, identity) follow the same rule.
#include "elementwise.cuh"

namespace rmlk {

template <typename O>
struct CastF {
    template <typename I>
    __device__ static O apply(I x) {
        if constexpr (std::is_same<O, bool>::value) {
            if constexpr (std::is_same<I, __half>::value)
                return __half2float(x) == 0.0f ? false : true;
            else
                return x == I(0) ? false : true;
        } else if constexpr (std::is_same<I, __half>::value && std::is_same<O, __half>::value) {
            return x;
        } else if constexpr (std::is_same<I, __half>::value) {
            return static_cast<O>(__half2float(x));
        } else if constexpr (std::is_same<O, __half>::value) {
            return __float2half(static_cast<float>(x));
        } else {
            return static_cast<O>(x);
        }
    }
};

template <typename I>
static int cast_dst(cudaStream_t st, int dst, size_t n, const void* in, void* out) {
    const int64_t shape[1] = {static_cast<int64_t>(n)};
    const int64_t s[1] = {1};
#define RMLK_CASE(DT, O) \
    case DT:             \
        return ew_launch1<CastF<O>, O, I>(st, 1, shape, s, static_cast<const I*>(in), static_cast<O*>(out));
    switch (dst) {
        RMLK_CASE(RMLK_F16, __half)
        RMLK_CASE(RMLK_F32, float)
        RMLK_CASE(RMLK_F64, double)
        RMLK_CASE(RMLK_I8, int8_t)
        RMLK_CASE(RMLK_U8, uint8_t)
        RMLK_CASE(RMLK_I16, int16_t)
        RMLK_CASE(RMLK_U16, uint16_t)
        RMLK_CASE(RMLK_I32, int32_t)
        RMLK_CASE(RMLK_U32, uint32_t)
        RMLK_CASE(RMLK_I64, int64_t)
        RMLK_CASE(RMLK_U64, uint64_t)
        RMLK_CASE(RMLK_BOOL, bool)
        default:
            return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported cast destination data type");
    }
#undef RMLK_CASE
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_cast(rmlk_stream_t stream, int src_dtype, int dst_dtype, size_t n, const void* in, void* out) {
    if (n == 0) return RMLK_OK;
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "cast: NULL tensor pointer");
    cudaStream_t st = as_stream(stream);
    switch (src_dtype) {
        case RMLK_F16: return cast_dst<__half>(st, dst_dtype, n, in, out);
        case RMLK_F32: return cast_dst<float>(st, dst_dtype, n, in, out);
        case RMLK_F64: return cast_dst<double>(st, dst_dtype, n, in, out);
        case RMLK_I8: return cast_dst<int8_t>(st, dst_dtype, n, in, out);
        case RMLK_U8: return cast_dst<uint8_t>(st, dst_dtype, n, in, out);
        case RMLK_I16: return cast_dst<int16_t>(st, dst_dtype, n, in, out);
        case RMLK_U16: return cast_dst<uint16_t>(st, dst_dtype, n, in, out);
        case RMLK_I32: return cast_dst<int32_t>(st, dst_dtype, n, in, out);
        case RMLK_U32: return cast_dst<uint32_t>(st, dst_dtype, n, in, out);
        case RMLK_I64: return cast_dst<int64_t>(st, dst_dtype, n, in, out);
        case RMLK_U64: return cast_dst<uint64_t>(st, dst_dtype, n, in, out);
        case RMLK_BOOL: return cast_dst<bool>(st, dst_dtype, n, in, out);
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported cast source data type");
    }
}
