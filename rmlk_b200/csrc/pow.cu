// Pow launcher: 5 base types x 11 exponent types, output in the base type.
//
// The arithmetic per pair is the reference's (cuda/src/ptx/pow.cu:6-65): f16 / f32 bases evaluate
// powf(float(x), float(y)); f64 bases pow(x, double(y)); integer bases
// (T)llround(pow(double(x), double(y))).  The same CUDA libm entry points are called, so results are
// bit-identical to the reference's kernels on the same GPU.
#include "elementwise.cuh"

namespace rmlk {

template <typename T> __device__ __forceinline__ float to_f32(T v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float to_f32<__half>(__half v) { return __half2float(v); }
template <typename T> __device__ __forceinline__ double to_f64(T v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ double to_f64<__half>(__half v) { return static_cast<double>(__half2float(v)); }

struct PowF {
    template <typename E> __device__ static __half apply(__half x, E y) { return __float2half(powf(__half2float(x), to_f32(y))); }
    template <typename E> __device__ static float apply(float x, E y) { return powf(x, to_f32(y)); }
    template <typename E> __device__ static double apply(double x, E y) { return pow(x, to_f64(y)); }
    template <typename E> __device__ static int32_t apply(int32_t x, E y) {
        return static_cast<int32_t>(llround(pow(static_cast<double>(x), to_f64(y))));
    }
    template <typename E> __device__ static int64_t apply(int64_t x, E y) {
        return static_cast<int64_t>(llround(pow(static_cast<double>(x), to_f64(y))));
    }
};

template <typename B>
static int pow_exp(cudaStream_t st, int exp_dtype, int rank, const int64_t* shape, const int64_t* as, const int64_t* bs,
                   const void* a, const void* b, void* out) {
#define RMLK_CASE(DT, E)                                                                                        \
    case DT:                                                                                                    \
        return ew_launch2<PowF, B, B, E>(st, rank, shape, as, bs, static_cast<const B*>(a), static_cast<const E*>(b), \
                                         static_cast<B*>(out));
    switch (exp_dtype) {
        RMLK_CASE(RMLK_U8, uint8_t)
        RMLK_CASE(RMLK_U16, uint16_t)
        RMLK_CASE(RMLK_U32, uint32_t)
        RMLK_CASE(RMLK_U64, uint64_t)
        RMLK_CASE(RMLK_I8, int8_t)
        RMLK_CASE(RMLK_I16, int16_t)
        RMLK_CASE(RMLK_I32, int32_t)
        RMLK_CASE(RMLK_I64, int64_t)
        RMLK_CASE(RMLK_F16, __half)
        RMLK_CASE(RMLK_F32, float)
        RMLK_CASE(RMLK_F64, double)
        default:
            return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported exponent data type for pow");
    }
#undef RMLK_CASE
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_pow(rmlk_stream_t stream, int base_dtype, int exp_dtype, int rank, const int64_t* shape,
                             const int64_t* a_strides, const int64_t* b_strides, const void* base,
                             const void* exponent, void* out) {
    if (int rc = ew_validate(rank, shape)) return rc;
    if (!base || !exponent || !out) return fail(RMLK_ERR_INVALID_ARG, "pow: NULL tensor pointer");
    if (rank > 0 && (!a_strides || !b_strides)) return fail(RMLK_ERR_INVALID_ARG, "pow: NULL strides");
    cudaStream_t st = as_stream(stream);
    switch (base_dtype) {
        case RMLK_F16: return pow_exp<__half>(st, exp_dtype, rank, shape, a_strides, b_strides, base, exponent, out);
        case RMLK_F32: return pow_exp<float>(st, exp_dtype, rank, shape, a_strides, b_strides, base, exponent, out);
        case RMLK_F64: return pow_exp<double>(st, exp_dtype, rank, shape, a_strides, b_strides, base, exponent, out);
        case RMLK_I32: return pow_exp<int32_t>(st, exp_dtype, rank, shape, a_strides, b_strides, base, exponent, out);
        case RMLK_I64: return pow_exp<int64_t>(st, exp_dtype, rank, shape, a_strides, b_strides, base, exponent, out);
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported base data type for pow");
    }
}
