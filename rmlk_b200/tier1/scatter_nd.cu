// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/scatter_nd.cu.
#include "t1_common.cuh"

#define T1_SCATTER(T, NAME, EXPR)                                                                                                    \
    struct NAME##_op {                                                                                                               \
        __device__ __forceinline__ T operator()(T in, T out) const { return EXPR; }                                                  \
    };                                                                                                                               \
    extern "C" __global__ void NAME(const size_t num_idx_tuples, const size_t data_len, const size_t data_rank,                      \
                                    const size_t indices_rank, const size_t updates_rank, const size_t* info,                        \
                                    const int64_t* indices, const T* updates, T* output, int* error) {                               \
        t1::scatter_nd_body(num_idx_tuples, data_len, data_rank, indices_rank, updates_rank, info, indices, updates, output, error,  \
                            NAME##_op());                                                                                            \
    }
#define T1_SCATTER_ALL(T, TAG, ADD, MUL)                                                                  \
    T1_SCATTER(T, scatter_nd_fwd_##TAG, in)                                                               \
    T1_SCATTER(T, scatter_nd_add_fwd_##TAG, ADD)                                                          \
    T1_SCATTER(T, scatter_nd_mul_fwd_##TAG, MUL)                                                          \
    T1_SCATTER(T, scatter_nd_max_fwd_##TAG, in > out ? in : out)                                          \
    T1_SCATTER(T, scatter_nd_min_fwd_##TAG, in < out ? in : out)

T1_SCATTER_ALL(__half, f16, __hadd(in, out), __hmul(in, out))
T1_SCATTER_ALL(float, f32, in + out, in * out)
T1_SCATTER_ALL(double, f64, in + out, in * out)
T1_SCATTER_ALL(int32_t, i32, in + out, in * out)
T1_SCATTER_ALL(int64_t, i64, in + out, in * out)
