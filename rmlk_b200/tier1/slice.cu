// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/slice.cu.
#include "t1_common.cuh"

#define T1_SLICE(T, I, NAME)                                                                                                      \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t axes_len, const size_t rank, const size_t* info,        \
                                    const T* input, const I* starts, const I* ends, const I* axes, const I* steps, T* output) {   \
        t1::slice_body(num_elems, axes_len, rank, info, input, starts, ends, axes, steps, output);                               \
    }

T1_SLICE(__half, int32_t, slice_fwd_f16_with_index_i32)
T1_SLICE(__half, int64_t, slice_fwd_f16_with_index_i64)
T1_SLICE(float, int32_t, slice_fwd_f32_with_index_i32)
T1_SLICE(float, int64_t, slice_fwd_f32_with_index_i64)
T1_SLICE(double, int32_t, slice_fwd_f64_with_index_i32)
T1_SLICE(double, int64_t, slice_fwd_f64_with_index_i64)
T1_SLICE(int32_t, int32_t, slice_fwd_i32_with_index_i32)
T1_SLICE(int32_t, int64_t, slice_fwd_i32_with_index_i64)
T1_SLICE(int64_t, int32_t, slice_fwd_i64_with_index_i32)
T1_SLICE(int64_t, int64_t, slice_fwd_i64_with_index_i64)
