// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/expand.cu.
#include "t1_common.cuh"

#define T1_EXPAND(T, NAME)                                                                                                         \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t input_rank, const size_t output_rank, const size_t* info, \
                                    const T* input, T* output) {                                                                   \
        t1::expand_body(num_elems, input_rank, output_rank, info, input, output);                                                  \
    }

T1_EXPAND(__half, expand_fwd_f16)
T1_EXPAND(float, expand_fwd_f32)
T1_EXPAND(double, expand_fwd_f64)
T1_EXPAND(int32_t, expand_fwd_i32)
T1_EXPAND(uint32_t, expand_fwd_u32)
T1_EXPAND(int64_t, expand_fwd_i64)
T1_EXPAND(uint64_t, expand_fwd_u64)
