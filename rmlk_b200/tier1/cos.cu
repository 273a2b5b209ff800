// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/cos.cu.
#include "t1_common.cuh"

#define T1_UNARY(T, NAME, EXPR)                                                           \
    struct NAME##_op {                                                                    \
        __device__ __forceinline__ T operator()(T x) const { return EXPR; }               \
    };                                                                                    \
    extern "C" __global__ void NAME(const size_t num_elems, const T* in, T* out) {        \
        t1::unary_body(num_elems, in, out, NAME##_op());                                  \
    }

T1_UNARY(__half, cos_fwd_f16, __float2half(cosf(__half2float(x))))
T1_UNARY(float, cos_fwd_f32, cosf(x))
T1_UNARY(double, cos_fwd_f64, cos(x))
