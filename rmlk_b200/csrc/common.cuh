// Shared device/host utilities for the rmlk_b200 kernels (sm_100a).
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdio>
#include <cstring>
#include <string>
#include <type_traits>

#include "../../include/rmlk_b200.h"

namespace rmlk {

// ---------------------------------------------------------------------------------------------
// error reporting
// ---------------------------------------------------------------------------------------------
void set_last_error(const std::string& msg);
int fail(int code, const std::string& msg);
int cuda_fail(cudaError_t e, const char* what);

#define RMLK_CHECK_LAUNCH(what)                                  \
    do {                                                         \
        cudaError_t _e = cudaGetLastError();                     \
        if (_e != cudaSuccess) return ::rmlk::cuda_fail(_e, what); \
    } while (0)

#define RMLK_CUDA(call)                                           \
    do {                                                          \
        cudaError_t _e = (call);                                  \
        if (_e != cudaSuccess) return ::rmlk::cuda_fail(_e, #call); \
    } while (0)

// Number of SMs of the current device (cached per device; an immutable capability table).
int sm_count();

// ---------------------------------------------------------------------------------------------
// Programmatic dependent launch.  Consecutive kernels of one stream normally run strictly one after the other:
// the next grid is scheduled only when the previous one has drained, and each small launch pays that gap.
// A kernel launched through launch_dep may be scheduled as soon as every CTA of the previous kernel has called
// dep_trigger() (or exited); it must then call dep_wait() before its first access to global memory, which blocks
// until the previous grid has completed and its writes are visible.  Kernels here call both at their very top,
// so that only scheduling and launch latency overlap, never memory accesses: ordering is exactly stream order.
// Both calls do nothing for a kernel launched the ordinary way.  RMLK_B200_NO_PDL=1 launches everything the
// ordinary way.
// ---------------------------------------------------------------------------------------------
bool dep_launch_enabled();

#ifdef __CUDACC__
__device__ __forceinline__ void dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void dep_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
// the usual opening of a kernel: let the next kernel be scheduled, then wait for the previous one
__device__ __forceinline__ void dep_sync() {
    dep_trigger();
    dep_wait();
}

template <typename... KArgs, typename... Args>
inline cudaError_t launch_dep(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    at[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = at;
    // Only grids of a few waves: there the launch gap is a visible share of the kernel.  A grid of hundreds of
    // thousands of small CTAs gains nothing from being scheduled early and measured slower with the attribute set
    // (a 64 M-element Range: 271 us against 137 us).
    const unsigned long long ctas = static_cast<unsigned long long>(grid.x) * grid.y * grid.z;
    cfg.numAttrs = (dep_launch_enabled() && ctas <= 32ull * static_cast<unsigned>(sm_count())) ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}
#endif

inline size_t dtype_size(int dt) {
    switch (dt) {
        case RMLK_F16: case RMLK_U16: case RMLK_I16: return 2;
        case RMLK_F32: case RMLK_I32: case RMLK_U32: return 4;
        case RMLK_F64: case RMLK_I64: case RMLK_U64: return 8;
        case RMLK_U8: case RMLK_I8: case RMLK_BOOL: return 1;
        default: return 0;
    }
}

// ---------------------------------------------------------------------------------------------
// 32-bit fast division (valid for dividends < 2^31), in the style of the well-known
// multiply-high + shift scheme: q = umulhi(n, mul) >> shr for d != 1.
// ---------------------------------------------------------------------------------------------
struct FastDiv {
    uint32_t d, mul, shr;
    FastDiv() : d(1), mul(0), shr(0) {}
    explicit FastDiv(uint32_t div) : d(div), mul(0), shr(0) {
        if (div > 1) {
            uint32_t lg = 0;
            while ((1ull << lg) < div) lg++;
            const uint32_t p = 31 + lg;
            mul = static_cast<uint32_t>(((1ull << p) + div - 1) / div);
            shr = p - 32;
        }
    }
    __host__ __device__ __forceinline__ uint32_t div(uint32_t n) const {
#ifdef __CUDA_ARCH__
        return d == 1 ? n : (__umulhi(n, mul) >> shr);
#else
        return d == 1 ? n : static_cast<uint32_t>((static_cast<uint64_t>(n) * mul) >> 32) >> shr;
#endif
    }
    __host__ __device__ __forceinline__ void divmod(uint32_t n, uint32_t& q, uint32_t& r) const {
        q = div(n);
        r = n - q * d;
    }
};

// ---------------------------------------------------------------------------------------------
// aligned element packs: the compiler emits one 128-bit access per 16 bytes
// ---------------------------------------------------------------------------------------------
template <typename T, int N>
struct alignas((sizeof(T) * N) >= 16 ? 16 : (sizeof(T) * N)) Pack {
    T v[N];
};

template <typename T, int N>
__device__ __forceinline__ Pack<T, N> load_pack(const T* p) {
    return *reinterpret_cast<const Pack<T, N>*>(p);
}
template <typename T, int N>
__device__ __forceinline__ void store_pack(T* p, const Pack<T, N>& v) {
    *reinterpret_cast<Pack<T, N>*>(p) = v;
}

// Streaming (read-once) 128-bit load that does not allocate in L1.
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}

template <int BYTES>
struct BytesT;
template <> struct BytesT<1> { using type = uint8_t; };
template <> struct BytesT<2> { using type = uint16_t; };
template <> struct BytesT<4> { using type = uint32_t; };
template <> struct BytesT<8> { using type = uint64_t; };
template <> struct BytesT<16> { using type = uint4; };

inline bool aligned_to(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

inline int64_t ceil_div64(int64_t a, int64_t b) { return (a + b - 1) / b; }

// Grid size for a flat kernel: enough blocks to cover `items`, capped so the grid stays a modest
// multiple of the SM count (the kernels are grid-stride).
inline unsigned flat_grid(int64_t items, int block, int per_sm_blocks) {
    int64_t need = ceil_div64(items, block);
    int64_t cap = static_cast<int64_t>(sm_count()) * per_sm_blocks;
    if (need < 1) need = 1;
    return static_cast<unsigned>(need < cap ? need : cap);
}

// Column-split MatMul across GPUs: other ranks' output buffers (mapped into this GPU's address space) that receive every
// element of C as well as the local one.
struct TcPeers {
    int n_peer;
    float* out[7];
    int64_t ldc;  // elements between rows of C in every destination
};

inline cudaStream_t as_stream(rmlk_stream_t s) { return reinterpret_cast<cudaStream_t>(s); }

}  // namespace rmlk
