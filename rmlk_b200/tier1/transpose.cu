// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/transpose.cu.
#include "t1_common.cuh"

#define T1_TRANSPOSE(T, NAME)                                                                                                  \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t rank, const size_t* info, const size_t* perm,         \
                                    const T* src_data, T* dst_data) {                                                          \
        t1::transpose_body(num_elems, rank, info, perm, src_data, dst_data);                                                   \
    }

T1_TRANSPOSE(__half, transpose_fwd_f16)
T1_TRANSPOSE(float, transpose_fwd_f32)
T1_TRANSPOSE(double, transpose_fwd_f64)
T1_TRANSPOSE(int32_t, transpose_fwd_i32)
T1_TRANSPOSE(int64_t, transpose_fwd_i64)
