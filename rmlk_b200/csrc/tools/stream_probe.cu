// Streaming micro-benchmark: how fast can a [K, N] fp32 weight matrix be pulled into shared memory, by access pattern.
// No arithmetic.  Every mbarrier wait is bounded (an error flag ends the run).  Usage: stream_probe K N [reps]
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <vector>

#define CK(x) do { cudaError_t e_ = (x); if (e_ != cudaSuccess) { printf("CUDA error %s at %s:%d\n", cudaGetErrorString(e_), __FILE__, __LINE__); exit(1); } } while (0)

constexpr uint32_t SPIN = 1u << 24;
__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory"); }
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory"); }
__device__ __forceinline__ void mbar_arrive(uint32_t bar) { asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory"); }
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, int* err) {
    for (uint32_t i = 0; i < SPIN; i++)
        if (mbar_try_wait(bar, parity)) return true;
    atomicExch(err, 1);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar) : "memory");
}
__device__ __forceinline__ void bulk_load_1d(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory");
}

// mode 0: row-major W, four [32 k][32 n] boxes per k-block (what the GEMM does)
// mode 1: row-major W, one [32 k][128 n] box per k-block
// mode 2: tile-major W (tile t = 128 columns, stored as [K][128] contiguous), one [32][128] box = 16 KB contiguous
// mode 3: tile-major W, one 16 KB 1-D bulk copy per k-block
// mode 4: row-major W, [32 k][256 n] tiles (two 128-wide boxes; half as many tiles)
// Work: items = tiles * kblocks; CTA c of G takes items [c * per, (c+1) * per) (stream-K style) when balanced = 1,
// else CTA = (tile, split) as the GEMM does (grid = tiles * ksplit).
struct P {
    int mode, kblocks, tiles, ksplit, balanced, stage_bytes;
    const float* w;
    int64_t N, K;
    int* err;
    float* sink;
};

template <int STAGES>
__global__ void __launch_bounds__(128, 1) stream_kernel(const __grid_constant__ CUtensorMap tm, P p) {
    extern __shared__ uint8_t raw[];
    const uint32_t base = (smem_u32(raw) + 1023u) & ~1023u;
    __shared__ uint64_t bars[2 * STAGES];
    const uint32_t full0 = smem_u32(&bars[0]), empty0 = smem_u32(&bars[STAGES]);
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) { mbar_init(full0 + 8 * s, 1); mbar_init(empty0 + 8 * s, 1); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    int64_t begin, end;  // item range; item = tile * kblocks + kb
    if (p.balanced) {
        const int64_t items = static_cast<int64_t>(p.tiles) * p.kblocks;
        const int64_t per = (items + gridDim.x - 1) / gridDim.x;
        begin = blockIdx.x * per;
        end = begin + per < items ? begin + per : items;
    } else {
        const int tile = blockIdx.x / p.ksplit, split = blockIdx.x % p.ksplit;
        const int per = (p.kblocks + p.ksplit - 1) / p.ksplit;
        const int kb0 = split * per, kb1 = kb0 + per < p.kblocks ? kb0 + per : p.kblocks;
        begin = static_cast<int64_t>(tile) * p.kblocks + kb0;
        end = static_cast<int64_t>(tile) * p.kblocks + kb1;
    }
    const int n_items = static_cast<int>(end > begin ? end - begin : 0);
    const int wide = p.mode == 4 ? 256 : 128;
    if (threadIdx.x == 0) {
        for (int it = 0; it < n_items; it++) {
            const int s = it % STAGES;
            if (it >= STAGES && !mbar_wait(empty0 + 8 * s, ((it / STAGES) - 1) & 1, p.err)) break;
            const int64_t item = begin + it;
            const int tile = static_cast<int>(item / p.kblocks), kb = static_cast<int>(item % p.kblocks);
            const uint32_t dst = base + s * p.stage_bytes;
            mbar_expect_tx(full0 + 8 * s, 32u * wide * 4u);
            if (p.mode == 0) {
                for (int j = 0; j < 4; j++) tma_load_2d(dst + j * 4096, &tm, tile * 128 + 32 * j, kb * 32, full0 + 8 * s);
            } else if (p.mode == 1) {
                tma_load_2d(dst, &tm, tile * 128, kb * 32, full0 + 8 * s);
            } else if (p.mode == 2) {
                tma_load_2d(dst, &tm, 0, static_cast<int>(static_cast<int64_t>(tile) * p.K + kb * 32), full0 + 8 * s);
            } else if (p.mode == 3) {
                bulk_load_1d(dst, p.w + (static_cast<int64_t>(tile) * p.K + kb * 32) * 128, 16384u, full0 + 8 * s);
            } else {
                tma_load_2d(dst, &tm, tile * 256, kb * 32, full0 + 8 * s);
                tma_load_2d(dst + 16384, &tm, tile * 256 + 128, kb * 32, full0 + 8 * s);
            }
        }
    } else if (threadIdx.x == 32) {
        float acc = 0.f;
        for (int it = 0; it < n_items; it++) {
            const int s = it % STAGES;
            if (!mbar_wait(full0 + 8 * s, (it / STAGES) & 1, p.err)) break;
            acc += *reinterpret_cast<const float*>(raw + (base - smem_u32(raw)) + s * p.stage_bytes);
            mbar_arrive(empty0 + 8 * s);
        }
        if (acc == 123.456f) *p.sink = acc;
    }
}

// plain vector loads, grid-stride, for reference
__global__ void __launch_bounds__(256) ldg_kernel(const float4* __restrict__ w, int64_t n4, float* sink) {
    float acc = 0.f;
    const int64_t stride = static_cast<int64_t>(gridDim.x) * 256 * 4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 * 4 + threadIdx.x; i < n4; i += stride) {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; u++) v[u] = i + u * 256 < n4 ? __ldcs(w + i + u * 256) : make_float4(0, 0, 0, 0);
#pragma unroll
        for (int u = 0; u < 4; u++) acc += v[u].x + v[u].y + v[u].z + v[u].w;
    }
    if (acc == 123.456f) *sink = acc;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*, const cuuint32_t*,
                                  const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn enc;
static void make_map(CUtensorMap* m, const void* ptr, uint64_t inner, uint64_t outer, uint32_t bi, uint32_t bo) {
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * 4};
    const cuuint32_t box[2] = {bi, bo};
    const cuuint32_t es[2] = {1, 1};
    CUresult r = enc(m, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, es, CU_TENSOR_MAP_INTERLEAVE_NONE,
                     CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) { printf("encode failed %d\n", (int)r); exit(1); }
}

template <int STAGES>
static float run(int mode, int64_t K, int64_t N, int ksplit, int balanced, int grid_override, std::vector<float*>& ring, int* err, float* sink, int reps) {
    const int wide = mode == 4 ? 256 : 128;
    P p;
    p.mode = mode; p.kblocks = static_cast<int>(K / 32); p.tiles = static_cast<int>(N / wide); p.ksplit = ksplit; p.balanced = balanced;
    p.stage_bytes = 32 * wide * 4; p.N = N; p.K = K; p.err = err; p.sink = sink;
    const int grid = balanced ? grid_override : p.tiles * ksplit;
    const size_t smem = static_cast<size_t>(STAGES) * p.stage_bytes + 1024;
    CK(cudaFuncSetAttribute(stream_kernel<STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(smem)));
    std::vector<CUtensorMap> maps(ring.size());
    for (size_t i = 0; i < ring.size(); i++) {
        if (mode == 0) make_map(&maps[i], ring[i], N, K, 32, 32);
        else if (mode == 1 || mode == 4) make_map(&maps[i], ring[i], N, K, 128, 32);
        else make_map(&maps[i], ring[i], 128, static_cast<uint64_t>(K) * (N / 128), 128, 32);
    }
    cudaEvent_t e0, e1;
    CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
    for (int i = 0; i < 3; i++) { p.w = ring[i % ring.size()]; stream_kernel<STAGES><<<grid, 128, smem>>>(maps[i % ring.size()], p); }
    CK(cudaDeviceSynchronize());
    CK(cudaEventRecord(e0));
    for (int i = 0; i < reps; i++) { p.w = ring[i % ring.size()]; stream_kernel<STAGES><<<grid, 128, smem>>>(maps[i % ring.size()], p); }
    CK(cudaEventRecord(e1));
    CK(cudaDeviceSynchronize());
    float ms;
    CK(cudaEventElapsedTime(&ms, e0, e1));
    return ms / reps * 1e3f;
}

int main(int argc, char** argv) {
    const int64_t K = argc > 1 ? atoll(argv[1]) : 2048, N = argc > 2 ? atoll(argv[2]) : 8192;
    const int reps = argc > 3 ? atoi(argv[3]) : 20;
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    CK(cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fp, cudaEnableDefault, &q));
    enc = reinterpret_cast<EncodeTiledFn>(fp);
    const size_t bytes = static_cast<size_t>(K) * N * 4;
    const int nring = bytes > (400u << 20) ? 2 : 6;
    std::vector<float*> ring(nring);
    for (auto& r : ring) { CK(cudaMalloc(&r, bytes)); CK(cudaMemset(r, 0, bytes)); }
    int* err; float* sink;
    CK(cudaMalloc(&err, 4)); CK(cudaMemset(err, 0, 4)); CK(cudaMalloc(&sink, 4));
    const double mb = bytes / 1e6;
    printf("K=%lld N=%lld  %.1f MB, ring %d\n", (long long)K, (long long)N, mb, nring);
    // LDG reference
    {
        cudaEvent_t e0, e1; CK(cudaEventCreate(&e0)); CK(cudaEventCreate(&e1));
        for (int g : {148 * 4, 148 * 8, 148 * 16}) {
            for (int i = 0; i < 3; i++) ldg_kernel<<<g, 256>>>(reinterpret_cast<const float4*>(ring[i % nring]), bytes / 16, sink);
            CK(cudaEventRecord(e0));
            for (int i = 0; i < reps; i++) ldg_kernel<<<g, 256>>>(reinterpret_cast<const float4*>(ring[i % nring]), bytes / 16, sink);
            CK(cudaEventRecord(e1)); CK(cudaDeviceSynchronize());
            float ms; CK(cudaEventElapsedTime(&ms, e0, e1));
            printf("ldg grid %5d: %7.1f us  %6.0f GB/s\n", g, ms / reps * 1e3, mb / (ms / reps) );
        }
    }
    const int tiles = static_cast<int>(N / 128);
    int ks = 148 / tiles; if (ks < 1) ks = 1; if (ks > K / 32 / 4) ks = static_cast<int>(K / 32 / 4);
    for (int mode = 0; mode <= 4; mode++) {
        for (int balanced = 0; balanced <= 1; balanced++) {
            const int ksplit = mode == 4 ? (2 * ks > 0 ? 2 * ks : 1) : ks;
            float t4 = run<4>(mode, K, N, ksplit, balanced, 148, ring, err, sink, reps);
            float t6 = mode == 4 ? 0.f : run<6>(mode, K, N, ksplit, balanced, 148, ring, err, sink, reps);
            float t12 = mode == 4 ? 0.f : run<12>(mode, K, N, ksplit, balanced, 148, ring, err, sink, reps);
            int h = 0; CK(cudaMemcpy(&h, err, 4, cudaMemcpyDeviceToHost));
            printf("mode %d %s ksplit %2d: 4 stages %7.1f us %6.0f GB/s | 6 stages %7.1f us %6.0f GB/s | 12 stages %7.1f us %6.0f GB/s  err=%d\n", mode,
                   balanced ? "balanced(148)" : "tile x split ", ksplit, t4, mb / t4 * 1e3, t6, t6 > 0 ? mb / t6 * 1e3 : 0.0, t12, t12 > 0 ? mb / t12 * 1e3 : 0.0, h);
            if (h) return 1;
        }
    }
    return 0;
}
