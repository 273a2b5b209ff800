// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/equal.cu.
#include "t1_common.cuh"

#define T1_BINARY(T, O, NAME, EXPR)                                                                                  \
    struct NAME##_op {                                                                                               \
        __device__ __forceinline__ O operator()(T x, T y) const { return EXPR; }                                     \
    };                                                                                                               \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t rank, const size_t* info, const T* a, const T* b, \
                                    O* out) {                                                                        \
        t1::binary_body(num_elems, rank, info, a, b, out, NAME##_op());                                              \
    }

T1_BINARY(__half, bool, equal_fwd_f16, x == y)
T1_BINARY(float, bool, equal_fwd_f32, x == y)
T1_BINARY(double, bool, equal_fwd_f64, x == y)
T1_BINARY(int32_t, bool, equal_fwd_i32, x == y)
T1_BINARY(int64_t, bool, equal_fwd_i64, x == y)
