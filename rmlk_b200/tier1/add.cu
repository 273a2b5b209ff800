// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/add.cu.
#include "t1_common.cuh"

#define T1_BINARY(T, O, NAME, EXPR)                                                                                  \
    struct NAME##_op {                                                                                               \
        __device__ __forceinline__ O operator()(T x, T y) const { return EXPR; }                                     \
    };                                                                                                               \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t rank, const size_t* info, const T* a, const T* b, \
                                    O* out) {                                                                        \
        t1::binary_body(num_elems, rank, info, a, b, out, NAME##_op());                                              \
    }

T1_BINARY(__half, __half, add_fwd_f16, x + y)
T1_BINARY(float, float, add_fwd_f32, x + y)
T1_BINARY(double, double, add_fwd_f64, x + y)
T1_BINARY(int32_t, int32_t, add_fwd_i32, x + y)
T1_BINARY(int64_t, int64_t, add_fwd_i64, x + y)

// b = alpha * a + beta * b, in place (same info layout)
#define T1_AXPBY(T, NAME)                                                                                                 \
    struct NAME##_op {                                                                                                    \
        __device__ __forceinline__ T operator()(T al, T x, T be, T y) const { return al * x + be * y; }                   \
    };                                                                                                                    \
    extern "C" __global__ void NAME(const T alpha, const T beta, const size_t num_elems, const size_t rank, const size_t* info, \
                                    const T* a, T* b) {                                                                   \
        t1::binary_inplace_body(alpha, beta, num_elems, rank, info, a, b, NAME##_op());                                   \
    }
T1_AXPBY(__half, add_alpha_beta_inplace_fwd_f16)
T1_AXPBY(float, add_alpha_beta_inplace_fwd_f32)
T1_AXPBY(double, add_alpha_beta_inplace_fwd_f64)
