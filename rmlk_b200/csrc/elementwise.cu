// Binary (Add/Sub/Mul/Div/Equal/Greater), unary (Sqrt/Neg/Sin/Cos/Sigmoid/Relu), Where, Expand and
// Fill launchers on the broadcast elementwise engine.
//
// Functor bodies use the same CUDA expressions as the reference's kernels so that results are
// bit-identical to them on the same GPU: `x + y`, `x / y` (IEEE, no fast-math), `sqrtf`, `sinf`,
// `cosf`, `x * -1` (reference cuda/src/ptx/{add,sub,mul,div,equal,greater,sqrt,neg,sin,cos,where}.cu).
#include "elementwise.cuh"

namespace rmlk {

struct AddF { template <typename T> __device__ static T apply(T x, T y) { return x + y; } };
struct SubF { template <typename T> __device__ static T apply(T x, T y) { return x - y; } };
struct MulF { template <typename T> __device__ static T apply(T x, T y) { return x * y; } };
struct DivF {
    template <typename T> __device__ static T apply(T x, T y) {
        if constexpr (std::is_integral<T>::value) {
            // Integer division by zero has no defined result in the reference either; return 0
            // instead of executing an undefined division.
            return y == 0 ? T(0) : (x / y);
        } else {
            return x / y;
        }
    }
};
struct EqF { template <typename T> __device__ static bool apply(T x, T y) { return x == y; } };
struct GtF { template <typename T> __device__ static bool apply(T x, T y) { return x > y; } };

struct SqrtF {
    __device__ static __half apply(__half x) { return hsqrt(x); }
    __device__ static float apply(float x) { return sqrtf(x); }
    __device__ static double apply(double x) { return sqrt(x); }
};
struct NegF {
    __device__ static __half apply(__half x) { return __hmul(x, __float2half(-1.0f)); }
    __device__ static float apply(float x) { return x * -1.0f; }
    __device__ static double apply(double x) { return x * -1.0; }
    __device__ static int32_t apply(int32_t x) { return x * -1; }
    __device__ static int64_t apply(int64_t x) { return x * -1; }
};
struct SinF {
    __device__ static __half apply(__half x) { return __float2half(sinf(__half2float(x))); }
    __device__ static float apply(float x) { return sinf(x); }
    __device__ static double apply(double x) { return sin(x); }
};
struct CosF {
    __device__ static __half apply(__half x) { return __float2half(cosf(__half2float(x))); }
    __device__ static float apply(float x) { return cosf(x); }
    __device__ static double apply(double x) { return cos(x); }
};
// Sigmoid: 1 / (1 + exp(-x)), the formula the reference checks its cuDNN result against
// (cuda/src/kernels/sigmoid.rs:37-39).
struct SigmoidF {
    __device__ static __half apply(__half x) { return __float2half(1.0f / (1.0f + expf(-__half2float(x)))); }
    __device__ static float apply(float x) { return 1.0f / (1.0f + expf(-x)); }
    __device__ static double apply(double x) { return 1.0 / (1.0 + exp(-x)); }
};
// Relu: max(x, 0) with NaN mapped to 0 (cuDNN NOT_PROPAGATE_NAN, cuda/src/kernels/relu.rs:25-27).
struct ReluF {
    __device__ static __half apply(__half x) { return x > __float2half(0.0f) ? x : __float2half(0.0f); }
    template <typename T> __device__ static T apply(T x) { return x > T(0) ? x : T(0); }
};
struct WhereF { template <typename T> __device__ static T apply(T x, T y, bool z) { return z ? x : y; } };
struct CopyF { template <typename T> __device__ static T apply(T x) { return x; } };

template <typename F, typename TO, typename T>
static int binary_typed(cudaStream_t st, int rank, const int64_t* shape, const int64_t* as, const int64_t* bs,
                        const void* a, const void* b, void* out) {
    return ew_launch2<F, TO, T, T>(st, rank, shape, as, bs, static_cast<const T*>(a), static_cast<const T*>(b),
                                   static_cast<TO*>(out));
}

template <typename F, bool TO_BOOL>
static int binary_dtype(cudaStream_t st, int dtype, int rank, const int64_t* shape, const int64_t* as,
                        const int64_t* bs, const void* a, const void* b, void* out) {
#define RMLK_CASE(DT, T)                                                                                   \
    case DT:                                                                                               \
        return binary_typed<F, typename std::conditional<TO_BOOL, bool, T>::type, T>(st, rank, shape, as, bs, a, \
                                                                                     b, out);
    switch (dtype) {
        RMLK_CASE(RMLK_F16, __half)
        RMLK_CASE(RMLK_F32, float)
        RMLK_CASE(RMLK_F64, double)
        RMLK_CASE(RMLK_I32, int32_t)
        RMLK_CASE(RMLK_I64, int64_t)
        default:
            return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for binary op");
    }
#undef RMLK_CASE
}

template <typename F, bool INTS>
static int unary_dtype(cudaStream_t st, int dtype, size_t n, const void* in, void* out) {
    const int64_t shape[1] = {static_cast<int64_t>(n)};
    const int64_t s[1] = {1};
    switch (dtype) {
        case RMLK_F16:
            return ew_launch1<F, __half, __half>(st, 1, shape, s, static_cast<const __half*>(in), static_cast<__half*>(out));
        case RMLK_F32:
            return ew_launch1<F, float, float>(st, 1, shape, s, static_cast<const float*>(in), static_cast<float*>(out));
        case RMLK_F64:
            return ew_launch1<F, double, double>(st, 1, shape, s, static_cast<const double*>(in), static_cast<double*>(out));
        case RMLK_I32:
            if constexpr (INTS)
                return ew_launch1<F, int32_t, int32_t>(st, 1, shape, s, static_cast<const int32_t*>(in), static_cast<int32_t*>(out));
            break;
        case RMLK_I64:
            if constexpr (INTS)
                return ew_launch1<F, int64_t, int64_t>(st, 1, shape, s, static_cast<const int64_t*>(in), static_cast<int64_t*>(out));
            break;
        default:
            break;
    }
    return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for unary op");
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_binary(rmlk_stream_t stream, int op, int dtype, int rank, const int64_t* shape,
                                const int64_t* a_strides, const int64_t* b_strides, const void* a, const void* b,
                                void* out) {
    if (int rc = ew_validate(rank, shape)) return rc;
    if (!a || !b || !out) return fail(RMLK_ERR_INVALID_ARG, "binary: NULL tensor pointer");
    if (rank > 0 && (!a_strides || !b_strides)) return fail(RMLK_ERR_INVALID_ARG, "binary: NULL strides");
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case RMLK_BIN_ADD: return binary_dtype<AddF, false>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        case RMLK_BIN_SUB: return binary_dtype<SubF, false>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        case RMLK_BIN_MUL: return binary_dtype<MulF, false>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        case RMLK_BIN_DIV: return binary_dtype<DivF, false>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        case RMLK_BIN_EQUAL: return binary_dtype<EqF, true>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        case RMLK_BIN_GREATER: return binary_dtype<GtF, true>(st, dtype, rank, shape, a_strides, b_strides, a, b, out);
        default: return fail(RMLK_ERR_INVALID_ARG, "binary: unknown op");
    }
}

extern "C" int rmlk_b200_unary(rmlk_stream_t stream, int op, int dtype, size_t n, const void* in, void* out) {
    if (n == 0) return RMLK_OK;
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "unary: NULL tensor pointer");
    cudaStream_t st = as_stream(stream);
    switch (op) {
        case RMLK_UN_SQRT: return unary_dtype<SqrtF, false>(st, dtype, n, in, out);
        case RMLK_UN_NEG: return unary_dtype<NegF, true>(st, dtype, n, in, out);
        case RMLK_UN_SIN: return unary_dtype<SinF, false>(st, dtype, n, in, out);
        case RMLK_UN_COS: return unary_dtype<CosF, false>(st, dtype, n, in, out);
        case RMLK_UN_SIGMOID: return unary_dtype<SigmoidF, false>(st, dtype, n, in, out);
        case RMLK_UN_RELU: return unary_dtype<ReluF, true>(st, dtype, n, in, out);
        default: return fail(RMLK_ERR_INVALID_ARG, "unary: unknown op");
    }
}

extern "C" int rmlk_b200_where(rmlk_stream_t stream, int dtype, int rank, const int64_t* shape,
                               const int64_t* x_strides, const int64_t* y_strides, const int64_t* cond_strides,
                               const void* x, const void* y, const void* cond, void* out) {
    if (int rc = ew_validate(rank, shape)) return rc;
    if (!x || !y || !cond || !out) return fail(RMLK_ERR_INVALID_ARG, "where: NULL tensor pointer");
    if (rank > 0 && (!x_strides || !y_strides || !cond_strides)) return fail(RMLK_ERR_INVALID_ARG, "where: NULL strides");
    cudaStream_t st = as_stream(stream);
    const bool* c = static_cast<const bool*>(cond);
#define RMLK_CASE(DT, T)                                                                                        \
    case DT:                                                                                                    \
        return ew_launch3<WhereF, T, T, T, bool>(st, rank, shape, x_strides, y_strides, cond_strides,           \
                                                 static_cast<const T*>(x), static_cast<const T*>(y), c, static_cast<T*>(out));
    switch (dtype) {
        RMLK_CASE(RMLK_F16, uint16_t)  // a select moves bits; no half arithmetic needed
        RMLK_CASE(RMLK_F32, uint32_t)
        RMLK_CASE(RMLK_I32, uint32_t)
        RMLK_CASE(RMLK_F64, uint64_t)
        RMLK_CASE(RMLK_I64, uint64_t)
        default:
            return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for where");
    }
#undef RMLK_CASE
}

// Expand whose broadcast dims form one block between a dense outer and a dense inner part
// (out[o][r][i] = in[o][i], e.g. grouped-query attention repeating each KV head R times): every 16-byte
// pack of the input is loaded once and stored R times, so the index arithmetic and the load are paid once
// per R stores.
__global__ void __launch_bounds__(256) expand_repeat_kernel(uint64_t in_packs, uint32_t inner_packs, FastDiv inner_div, uint32_t repeat,
                                                            const uint4* __restrict__ in, uint4* __restrict__ out) {
    dep_sync();
    const uint64_t idx = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (idx >= in_packs) return;
    uint64_t o;
    uint32_t i;
    if (in_packs <= 0x7fffffffull) {
        const uint32_t q = inner_div.div(static_cast<uint32_t>(idx));
        o = q;
        i = static_cast<uint32_t>(idx) - q * inner_packs;
    } else {
        o = idx / inner_packs;
        i = static_cast<uint32_t>(idx - o * inner_packs);
    }
    const uint4 v = ld_stream_u4(in + idx);
    uint4* dst = out + o * repeat * inner_packs + i;
    for (uint32_t r = 0; r < repeat; r++) dst[static_cast<uint64_t>(r) * inner_packs] = v;
}

extern "C" int rmlk_b200_expand(rmlk_stream_t stream, int elem_size, int in_rank, const int64_t* in_shape,
                                int out_rank, const int64_t* out_shape, const void* in, void* out) {
    if (int rc = ew_validate(out_rank, out_shape)) return rc;
    if (in_rank < 0 || in_rank > out_rank) return fail(RMLK_ERR_INVALID_ARG, "expand: input rank exceeds output rank");
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "expand: NULL tensor pointer");
    // Right-aligned broadcast strides: stride 0 where the input dim is 1 or missing
    // (reference cuda/src/ptx/headers/expand_op_macros.cuh:20-27).
    int64_t strides[RMLK_MAX_RANK] = {0};
    int64_t run = 1;
    for (int d = out_rank - 1; d >= 0; d--) {
        const int id = d - (out_rank - in_rank);
        if (id >= 0) {
            if (in_shape[id] != 1 && in_shape[id] != out_shape[d])
                return fail(RMLK_ERR_INVALID_ARG, "expand: incompatible shapes for broadcast");
            strides[d] = in_shape[id] == 1 ? 0 : run;
            run *= in_shape[id];
        } else {
            strides[d] = 0;
        }
    }
    cudaStream_t st = as_stream(stream);
    {
        // [dense outer] [broadcast block] [dense inner]?
        int64_t outer = 1, repeat = 1, inner = 1;
        int phase = 0;  // 0 outer, 1 broadcast, 2 inner
        bool one_block = true;
        for (int d = 0; d < out_rank && one_block; d++) {
            if (out_shape[d] == 1) continue;
            const bool bc = strides[d] == 0;
            if (phase == 0) {
                if (bc) { phase = 1; repeat *= out_shape[d]; } else outer *= out_shape[d];
            } else if (phase == 1) {
                if (bc) repeat *= out_shape[d]; else { phase = 2; inner *= out_shape[d]; }
            } else {
                if (bc) one_block = false; else inner *= out_shape[d];
            }
        }
        const int64_t inner_bytes = inner * elem_size;
        if (one_block && phase == 2 && repeat > 1 && repeat <= 64 && inner_bytes % 16 == 0 && inner_bytes / 16 <= 0x7fffffffll &&
            aligned_to(in, 16) && aligned_to(out, 16) && (elem_size == 1 || elem_size == 2 || elem_size == 4 || elem_size == 8)) {
            const uint64_t inner_packs = static_cast<uint64_t>(inner_bytes / 16);
            const uint64_t in_packs = static_cast<uint64_t>(outer) * inner_packs;
            if (in_packs == 0) return RMLK_OK;
            if (in_packs / 256 < 0x7fffffffull) {
                launch_dep(expand_repeat_kernel, dim3(static_cast<unsigned>((in_packs + 255) / 256)), dim3(256), 0, st, 
                    in_packs, static_cast<uint32_t>(inner_packs), FastDiv(static_cast<uint32_t>(inner_packs)), static_cast<uint32_t>(repeat),
                    static_cast<const uint4*>(in), static_cast<uint4*>(out));
                RMLK_CHECK_LAUNCH("expand_repeat_kernel");
                return RMLK_OK;
            }
        }
    }
    switch (elem_size) {
        case 1: return ew_launch1<CopyF, uint8_t, uint8_t>(st, out_rank, out_shape, strides, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out));
        case 2: return ew_launch1<CopyF, uint16_t, uint16_t>(st, out_rank, out_shape, strides, static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out));
        case 4: return ew_launch1<CopyF, uint32_t, uint32_t>(st, out_rank, out_shape, strides, static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out));
        case 8: return ew_launch1<CopyF, uint64_t, uint64_t>(st, out_rank, out_shape, strides, static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out));
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "expand: element size must be 1, 2, 4 or 8");
    }
}
