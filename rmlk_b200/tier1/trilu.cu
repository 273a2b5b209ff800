// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/trilu.cu.
#include "t1_common.cuh"

#define T1_TRILU(T, NAME)                                                                                              \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t rank, const bool upper, const int64_t k,     \
                                    const size_t* info, const T* input, T* output) {                                  \
        if (rank == 3) t1::trilu_body(num_elems, upper, k, info, input, output);                                      \
    }

T1_TRILU(__half, trilu_fwd_f16)
T1_TRILU(float, trilu_fwd_f32)
T1_TRILU(double, trilu_fwd_f64)
T1_TRILU(int32_t, trilu_fwd_i32)
T1_TRILU(uint32_t, trilu_fwd_u32)
T1_TRILU(int64_t, trilu_fwd_i64)
T1_TRILU(uint64_t, trilu_fwd_u64)
