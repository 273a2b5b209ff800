// Tier-1 (symbol-compatible) kernels: entry points of the reference module cuda/src/ptx/pow.cu.
#include "t1_common.cuh"

// f16 / f32 bases: powf in float; f64: pow in double; integer bases: llround(pow(double, double)), as the reference.
template <typename E> __device__ __forceinline__ float t1_f(E v) { return static_cast<float>(v); }
template <> __device__ __forceinline__ float t1_f<__half>(__half v) { return __half2float(v); }
template <typename E> __device__ __forceinline__ double t1_d(E v) { return static_cast<double>(v); }
template <> __device__ __forceinline__ double t1_d<__half>(__half v) { return static_cast<double>(__half2float(v)); }

#define T1_POW(B, BT, E, ET, EXPR)                                                                                          \
    struct pow_fwd_##BT##_##ET##_op {                                                                                       \
        __device__ __forceinline__ B operator()(B x, E y) const { return EXPR; }                                            \
    };                                                                                                                      \
    extern "C" __global__ void pow_fwd_##BT##_##ET(const size_t num_elems, const size_t rank, const size_t* info, const B* a, \
                                                   const E* b, B* out) {                                                      \
        t1::binary_body(num_elems, rank, info, a, b, out, pow_fwd_##BT##_##ET##_op());                                        \
    }
#define T1_POW_ALL_EXP(B, BT, EXPR)                                                                                                     \
    T1_POW(B, BT, uint8_t, u8, EXPR) T1_POW(B, BT, uint16_t, u16, EXPR) T1_POW(B, BT, uint32_t, u32, EXPR) T1_POW(B, BT, uint64_t, u64, EXPR) \
    T1_POW(B, BT, int8_t, i8, EXPR) T1_POW(B, BT, int16_t, i16, EXPR) T1_POW(B, BT, int32_t, i32, EXPR) T1_POW(B, BT, int64_t, i64, EXPR)     \
    T1_POW(B, BT, __half, f16, EXPR) T1_POW(B, BT, float, f32, EXPR) T1_POW(B, BT, double, f64, EXPR)

T1_POW_ALL_EXP(__half, f16, __float2half(powf(__half2float(x), t1_f(y))))
T1_POW_ALL_EXP(float, f32, powf(x, t1_f(y)))
T1_POW_ALL_EXP(double, f64, pow(x, t1_d(y)))
T1_POW_ALL_EXP(int32_t, i32, static_cast<int32_t>(llround(pow(static_cast<double>(x), t1_d(y)))))
T1_POW_ALL_EXP(int64_t, i64, static_cast<int64_t>(llround(pow(static_cast<double>(x), t1_d(y)))))
