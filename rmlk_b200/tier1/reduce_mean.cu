// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/reduce_mean.cu.
#include "t1_common.cuh"

// Sequential sum in double (floats) or uint64 (integers), mean in double, one thread per output element.
#define T1_REDUCE_MEAN(T, ACC, NAME, LOAD, STORE)                                                                              \
    struct NAME##_load {                                                                                                       \
        __device__ __forceinline__ ACC operator()(T x) const { return LOAD; }                                                  \
    };                                                                                                                         \
    struct NAME##_store {                                                                                                      \
        __device__ __forceinline__ T operator()(double m) const { return STORE; }                                              \
    };                                                                                                                         \
    extern "C" __global__ void NAME(const size_t* axes, const size_t num_axes, const size_t rank, const size_t* info,         \
                                    const T* input, const size_t reduced_dim_prod, const size_t num_out_elems, T* output) {   \
        t1::reduce_mean_body<T, ACC>(axes, num_axes, rank, info, input, reduced_dim_prod, num_out_elems, output, NAME##_load(), \
                                     NAME##_store());                                                                          \
    }

T1_REDUCE_MEAN(__half, double, reduce_mean_fwd_f16, static_cast<double>(__half2float(x)), __float2half(static_cast<float>(m)))
T1_REDUCE_MEAN(float, double, reduce_mean_fwd_f32, static_cast<double>(x), static_cast<float>(m))
T1_REDUCE_MEAN(double, double, reduce_mean_fwd_f64, x, m)
T1_REDUCE_MEAN(uint32_t, uint64_t, reduce_mean_fwd_u32, static_cast<uint64_t>(x), static_cast<uint32_t>(m))
T1_REDUCE_MEAN(uint64_t, uint64_t, reduce_mean_fwd_u64, x, static_cast<uint64_t>(m))
