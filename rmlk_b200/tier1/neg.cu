// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/neg.cu.
#include "t1_common.cuh"

#define T1_UNARY(T, NAME, EXPR)                                                           \
    struct NAME##_op {                                                                    \
        __device__ __forceinline__ T operator()(T x) const { return EXPR; }               \
    };                                                                                    \
    extern "C" __global__ void NAME(const size_t num_elems, const T* in, T* out) {        \
        t1::unary_body(num_elems, in, out, NAME##_op());                                  \
    }

T1_UNARY(__half, neg_fwd_f16, __hmul(x, __float2half(-1.0f)))
T1_UNARY(float, neg_fwd_f32, x * -1.0f)
T1_UNARY(double, neg_fwd_f64, x * -1.0)
T1_UNARY(int32_t, neg_fwd_i32, x * -1)
T1_UNARY(int64_t, neg_fwd_i64, x * -1)
