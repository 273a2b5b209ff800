// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/where.cu.
#include "t1_common.cuh"

#define T1_WHERE(T, NAME)                                                                                                    \
    extern "C" __global__ void NAME(const size_t num_elems, const size_t rank, const size_t* info, const T* x, const T* y,    \
                                    const bool* cond, T* out) {                                                              \
        t1::where_body(num_elems, rank, info, x, y, cond, out);                                                              \
    }

T1_WHERE(__half, where_fwd_f16)
T1_WHERE(float, where_fwd_f32)
T1_WHERE(double, where_fwd_f64)
T1_WHERE(int32_t, where_fwd_i32)
T1_WHERE(int64_t, where_fwd_i64)
