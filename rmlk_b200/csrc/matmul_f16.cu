// f16 MatMul: C[b] = A[b] x B[b], row-major, half in and out, products accumulated in fp32 and rounded to f16 once.
// The reference runs cublasGemmStridedBatchedEx with CUBLAS_COMPUTE_16F for f16 (cuda/src/params.rs:24-31,
// cuda/src/kernels/gemm.rs:206-231): same operands and result type, half-precision accumulation; this kernel's sums
// are at least as accurate.  Shared-memory tiled SIMT kernel (64 x 64 x 16, 256 threads, 4 x 4 micro-tiles, guarded
// edges, any M / N / K, batch strides may be 0 to broadcast an operand).  The benchmark path is fp32; a tensor-core
// kind::f16 kernel is not built.
#include "common.cuh"

namespace rmlk {

constexpr int HF_BM = 64, HF_BN = 64, HF_BK = 16;

__global__ void __launch_bounds__(256) gemm_f16_kernel(const __half* __restrict__ a, const __half* __restrict__ b, __half* __restrict__ c, int64_t M,
                                                      int64_t N, int64_t K, int64_t sa, int64_t sb, int64_t sc) {
    dep_sync();
    __shared__ float As[HF_BK][HF_BM + 4];
    __shared__ float Bs[HF_BK][HF_BN + 4];
    const int tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const int64_t batch = blockIdx.z;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * HF_BM, n0 = static_cast<int64_t>(blockIdx.x) * HF_BN;
    const __half* A = a + batch * sa;
    const __half* B = b + batch * sb;
    __half* C = c + batch * sc;
    float acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[i][j] = 0.f;
    for (int64_t k0 = 0; k0 < K; k0 += HF_BK) {
        // A tile: 64 rows x 16 k, consecutive threads along k; B tile: 16 k x 64 columns, consecutive threads along n
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int e = tid + 256 * i;
            const int row = e >> 4, kk = e & 15;
            const int64_t gm = m0 + row, gk = k0 + kk;
            As[kk][row] = (gm < M && gk < K) ? __half2float(A[gm * K + gk]) : 0.f;
            const int kr = e >> 6, col = e & 63;
            const int64_t gk2 = k0 + kr, gn = n0 + col;
            Bs[kr][col] = (gk2 < K && gn < N) ? __half2float(B[gk2 * N + gn]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < HF_BK; kk++) {
            float av[4], bv[4];
#pragma unroll
            for (int i = 0; i < 4; i++) av[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; j++) bv[j] = Bs[kk][tx * 4 + j];
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(av[i], bv[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int64_t gm = m0 + ty * 4 + i;
        if (gm >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int64_t gn = n0 + tx * 4 + j;
            if (gn < N) C[gm * N + gn] = __float2half_rn(acc[i][j]);
        }
    }
}

int matmul_f16(cudaStream_t st, int64_t batch, int64_t m, int64_t n, int64_t k, const void* a, int64_t sa, const void* b, int64_t sb, void* c,
               int64_t sc) {
    if (k == 0) {
        for (int64_t bi = 0; bi < batch; bi++)
            RMLK_CUDA(cudaMemsetAsync(static_cast<__half*>(c) + bi * sc, 0, static_cast<size_t>(m) * n * sizeof(__half), st));
        return RMLK_OK;
    }
    const int64_t gx = ceil_div64(n, HF_BN), gy = ceil_div64(m, HF_BM);
    if (gx > 0x7fffffffll || gy > 65535 || batch > 65535) return fail(RMLK_ERR_INVALID_ARG, "matmul f16: extent too large");
    launch_dep(gemm_f16_kernel, dim3(static_cast<unsigned>(gx), static_cast<unsigned>(gy), static_cast<unsigned>(batch)), dim3(256), 0, st,
               static_cast<const __half*>(a), static_cast<const __half*>(b), static_cast<__half*>(c), m, n, k, sa, sb, sc);
    RMLK_CHECK_LAUNCH("gemm_f16_kernel");
    return RMLK_OK;
}

}  // namespace rmlk
