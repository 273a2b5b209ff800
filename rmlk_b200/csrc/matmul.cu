// fp32 MatMul: C[b] = A[b] x B[b], row-major, fp32 accumulate.
//
// Two kernels, chosen by shape in rmlk_b200_matmul:
//
//  skinny_kernel   M <= 16 (decode GEMV / small-batch decode).  Memory-bound: every element of B is
//                  read exactly once with 128-bit loads along N; a CTA owns a 32-column strip and its
//                  256 threads are 8 column-quads x 32 k-lanes, 8 independent 128-bit loads in flight
//                  per thread.  The A rows of the current k-chunk are staged in shared memory as
//                  [k][m] so one LDS.128 feeds four FMAs rows.  When the strip count cannot fill the
//                  GPU, K is also split across CTAs into a caller-provided scratch buffer that a
//                  second kernel sums in a fixed order (deterministic, no atomics).
//
//  gemm_kernel     everything else.  Shared-memory tiled SIMT GEMM (BM x BN x 16, 256 threads,
//                  register micro-tiles, double-buffered) with guarded edges, any M/N/K.
//
// The reference calls cublasGemmStridedBatchedEx with CUBLAS_COMPUTE_32F
// (cuda/src/kernels/gemm.rs:206-231); both kernels accumulate in fp32 with FMA.
#include <atomic>

#include "common.cuh"

namespace rmlk {

// ---------------------------------------------------------------------------------------------
// skinny
// ---------------------------------------------------------------------------------------------
constexpr int SK_COLS = 32;    // columns per CTA
constexpr int SK_KC = 256;     // k-chunk staged in shared memory
constexpr int SK_THREADS = 256;

struct SkinnyParams {
    const float* a;
    const float* b;
    float* c;          // final output, or the split-K scratch when ksplit > 1
    int64_t M, N, K;
    int64_t sa, sb, sc;  // batch strides (elements)
    int64_t k_per_split;
    int ksplit;
    int vec_b;           // B rows are 16-byte aligned (N % 4 == 0 and base aligned)
};

template <int MB>
__global__ void __launch_bounds__(SK_THREADS) skinny_kernel(SkinnyParams p) {
    dep_sync();
    constexpr int SA = MB >= 8 ? MB + 4 : MB;  // padded row stride: fewer bank conflicts while staging
    __shared__ __align__(16) float sA[SK_KC * SA];
    __shared__ __align__(16) float sRed[8 * MB * SK_COLS];
    const int tx = threadIdx.x & 7;   // column quad
    const int ty = threadIdx.x >> 3;  // k lane 0..31
    const int64_t batch = blockIdx.z;
    const int split = blockIdx.y;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * SK_COLS + tx * 4;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb;
    const int64_t kbeg = static_cast<int64_t>(split) * p.k_per_split;
    const int64_t kend = kbeg + p.k_per_split < p.K ? kbeg + p.k_per_split : p.K;

    float acc[MB][4];
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;

    const bool full_cols = p.vec_b && (n0 + 3 < p.N);
    for (int64_t kc = kbeg; kc < kend; kc += SK_KC) {
        const int kn = static_cast<int>(kend - kc < SK_KC ? kend - kc : SK_KC);
        __syncthreads();
        // stage A[:, kc:kc+kn] as sA[k][m]
        for (int i = threadIdx.x; i < SK_KC * MB; i += SK_THREADS) {
            const int m = i / SK_KC, k = i - m * SK_KC;  // consecutive threads -> consecutive k (coalesced)
            float v = 0.f;
            if (m < p.M && k < kn) v = A[static_cast<int64_t>(m) * p.K + kc + k];
            sA[k * SA + m] = v;
        }
        __syncthreads();
        float4 bv[8];
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int k = ty + u * 32;
            bv[u] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (k < kn) {
                const float* src = B + (kc + k) * p.N + n0;
                if (full_cols) {
                    const uint4 raw = ld_stream_u4(src);
                    bv[u] = make_float4(__uint_as_float(raw.x), __uint_as_float(raw.y), __uint_as_float(raw.z), __uint_as_float(raw.w));
                } else {
                    if (n0 + 0 < p.N) bv[u].x = src[0];
                    if (n0 + 1 < p.N) bv[u].y = src[1];
                    if (n0 + 2 < p.N) bv[u].z = src[2];
                    if (n0 + 3 < p.N) bv[u].w = src[3];
                }
            }
        }
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int k = ty + u * 32;
            const float* arow = sA + k * SA;
            float av[MB];
            if constexpr (MB % 4 == 0) {
#pragma unroll
                for (int m = 0; m < MB; m += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(arow + m);
                    av[m] = t.x; av[m + 1] = t.y; av[m + 2] = t.z; av[m + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int m = 0; m < MB; m++) av[m] = arow[m];
            }
#pragma unroll
            for (int m = 0; m < MB; m++) {
                acc[m][0] = fmaf(av[m], bv[u].x, acc[m][0]);
                acc[m][1] = fmaf(av[m], bv[u].y, acc[m][1]);
                acc[m][2] = fmaf(av[m], bv[u].z, acc[m][2]);
                acc[m][3] = fmaf(av[m], bv[u].w, acc[m][3]);
            }
        }
    }
    // reduce the 32 k-lanes: 4 inside each warp by shuffle, 8 warps through shared memory
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float v = acc[m][j];
            v += __shfl_xor_sync(0xffffffffu, v, 8);
            v += __shfl_xor_sync(0xffffffffu, v, 16);
            acc[m][j] = v;
        }
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (lane < 8) {
#pragma unroll
        for (int m = 0; m < MB; m++)
#pragma unroll
            for (int j = 0; j < 4; j++) sRed[(warp * MB + m) * SK_COLS + lane * 4 + j] = acc[m][j];
    }
    __syncthreads();
    float* __restrict__ C = p.c + (p.ksplit > 1 ? (static_cast<int64_t>(split) * gridDim.z + batch) * p.M * p.N : batch * p.sc);
    for (int i = threadIdx.x; i < MB * SK_COLS; i += SK_THREADS) {
        const int m = i / SK_COLS, c = i - m * SK_COLS;
        const int64_t n = static_cast<int64_t>(blockIdx.x) * SK_COLS + c;
        if (m < p.M && n < p.N) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) s += sRed[(w * MB + m) * SK_COLS + c];
            C[static_cast<int64_t>(m) * p.N + n] = s;
        }
    }
}

// ---------------------------------------------------------------------------------------------
// wide-strip small-M MatMul (M <= 16, rows of B 16-byte aligned): the decode GEMV
// ---------------------------------------------------------------------------------------------
// Memory-bound: B is read exactly once.  A CTA owns a strip of 128 columns (a warp-wide load is one 512-byte piece
// of a row of B; 128-byte pieces stream a fifth slower) and a range of K; its 8 warps take rows k, k + 8, ... of the
// range, each thread holding 8 independent 128-bit loads in flight.  A round covers 64 rows of B: the loads go
// out first, then the 64 x MB block of A is staged in shared memory as [k][m] under them, then the FMAs.  K is split
// over enough CTAs to keep several per SM in flight (the partial sums go through the caller's scratch and the
// fixed-order split-K sum); a thread's 8 k-lanes are added by a three-step tree through shared memory.
constexpr int GW_COLS = 128;
constexpr int GW_U = 8;                 // loads in flight per thread
constexpr int GW_KR = 8 * GW_U;         // rows of B per round
constexpr int GW_THREADS = 256;

template <int MB>
__global__ void __launch_bounds__(GW_THREADS) gemv_wide_kernel(SkinnyParams p) {
    dep_sync();
    __shared__ __align__(16) float sA[GW_KR * MB];
    __shared__ __align__(16) float sRed[4 * MB * GW_COLS];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int64_t batch = blockIdx.z;
    const int split = blockIdx.y;
    const int64_t n0 = static_cast<int64_t>(blockIdx.x) * GW_COLS + lane * 4;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb;
    const int64_t kbeg = static_cast<int64_t>(split) * p.k_per_split;
    const int64_t kend = kbeg + p.k_per_split < p.K ? kbeg + p.k_per_split : p.K;
    const bool in_cols = n0 < p.N;  // N % 4 == 0: a column quad is inside or outside as a whole

    float acc[MB][4];
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;

    for (int64_t kc = kbeg; kc < kend; kc += GW_KR) {
        const int kn = static_cast<int>(kend - kc < GW_KR ? kend - kc : GW_KR);
        uint4 bv[GW_U];
#pragma unroll
        for (int u = 0; u < GW_U; u++) {
            const int k = warp + u * 8;
            bv[u] = make_uint4(0u, 0u, 0u, 0u);
            if (k < kn && in_cols) bv[u] = ld_stream_u4(B + (kc + k) * p.N + n0);
        }
        __syncthreads();  // the previous round's FMAs have read sA
        for (int i = threadIdx.x; i < GW_KR * MB; i += GW_THREADS) {
            const int m = i / GW_KR, k = i - m * GW_KR;  // consecutive threads -> consecutive k (coalesced)
            float v = 0.f;
            if (m < p.M && k < kn) v = A[static_cast<int64_t>(m) * p.K + kc + k];
            sA[k * MB + m] = v;
        }
        __syncthreads();
#pragma unroll
        for (int u = 0; u < GW_U; u++) {
            const float* arow = sA + (warp + u * 8) * MB;  // the same address across a warp: a broadcast
            float av[MB];
            if constexpr (MB % 4 == 0) {
#pragma unroll
                for (int m = 0; m < MB; m += 4) {
                    const float4 t = *reinterpret_cast<const float4*>(arow + m);
                    av[m] = t.x; av[m + 1] = t.y; av[m + 2] = t.z; av[m + 3] = t.w;
                }
            } else {
#pragma unroll
                for (int m = 0; m < MB; m++) av[m] = arow[m];
            }
            const float bx = __uint_as_float(bv[u].x), by = __uint_as_float(bv[u].y), bz = __uint_as_float(bv[u].z), bw = __uint_as_float(bv[u].w);
#pragma unroll
            for (int m = 0; m < MB; m++) {
                acc[m][0] = fmaf(av[m], bx, acc[m][0]);
                acc[m][1] = fmaf(av[m], by, acc[m][1]);
                acc[m][2] = fmaf(av[m], bz, acc[m][2]);
                acc[m][3] = fmaf(av[m], bw, acc[m][3]);
            }
        }
    }
    // add the 8 warps (k lanes): 4..7 into 0..3, 2..3 into 0..1, 1 into 0
#pragma unroll
    for (int half = 4; half >= 1; half >>= 1) {
        __syncthreads();
        if (warp >= half && warp < 2 * half) {
#pragma unroll
            for (int m = 0; m < MB; m++)
                *reinterpret_cast<float4*>(sRed + ((warp - half) * MB + m) * GW_COLS + lane * 4) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
        }
        __syncthreads();
        if (warp < half) {
#pragma unroll
            for (int m = 0; m < MB; m++) {
                const float4 t = *reinterpret_cast<const float4*>(sRed + (warp * MB + m) * GW_COLS + lane * 4);
                acc[m][0] += t.x; acc[m][1] += t.y; acc[m][2] += t.z; acc[m][3] += t.w;
            }
        }
    }
    if (warp == 0 && in_cols) {
        float* __restrict__ C = p.c + (p.ksplit > 1 ? (static_cast<int64_t>(split) * gridDim.z + batch) * p.M * p.N : batch * p.sc);
#pragma unroll
        for (int m = 0; m < MB; m++)
            if (m < p.M) *reinterpret_cast<float4*>(C + static_cast<int64_t>(m) * p.N + n0) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    }
}

// K split of the wide-strip kernel: about six CTAs per SM, ranges that are multiples of a round, and partial sums that
// stay below a tenth of the bytes of B.
static int gemv_wide_plan(int64_t batch, int64_t m, int64_t n, int64_t k, int64_t* k_per_split) {
    const int64_t strips = ceil_div64(n, GW_COLS) * batch;
    int64_t s = ceil_div64(6ll * sm_count(), strips);
    const int64_t by_traffic = k / (20 * m) > 0 ? k / (20 * m) : 1;
    if (s > by_traffic) s = by_traffic;
    const int64_t rounds = ceil_div64(k, GW_KR);
    if (s > rounds) s = rounds;
    if (s < 1) s = 1;
    if (s > 64) s = 64;
    *k_per_split = ceil_div64(rounds, s) * GW_KR;
    return static_cast<int>(ceil_div64(k, *k_per_split));
}

// Many small problems with a short K (decode attention scores: batch x heads problems of [1, 64] x [64, T]).
// One thread owns four adjacent columns of one problem and walks all of K itself: no shared memory, no
// reduction, B read once with 128-bit loads (a warp reads 512 contiguous bytes of a B row per k), A read with
// 128-bit loads that are the same address across the lanes of a problem.  Needs N % 4 == 0, K % 4 == 0 and
// 16-byte aligned operands and batch strides.
template <int MB>
__global__ void __launch_bounds__(256) smallk_kernel(SkinnyParams p, int64_t total_quads, uint32_t nq) {
    dep_sync();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (idx >= total_quads) return;
    const int64_t batch = idx / nq;
    const int64_t n0 = (idx - batch * nq) * 4;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb + n0;
    float acc[MB][4];
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;
    const int K = static_cast<int>(p.K);
#pragma unroll 4
    for (int k = 0; k < K; k += 4) {
        uint4 bv[4];
#pragma unroll
        for (int u = 0; u < 4; u++) bv[u] = ld_stream_u4(B + static_cast<int64_t>(k + u) * p.N);
#pragma unroll
        for (int m = 0; m < MB; m++) {
            if (m < p.M) {
                const float4 av = __ldg(reinterpret_cast<const float4*>(A + static_cast<int64_t>(m) * p.K + k));
                const float a4[4] = {av.x, av.y, av.z, av.w};
#pragma unroll
                for (int u = 0; u < 4; u++) {
                    acc[m][0] = fmaf(a4[u], __uint_as_float(bv[u].x), acc[m][0]);
                    acc[m][1] = fmaf(a4[u], __uint_as_float(bv[u].y), acc[m][1]);
                    acc[m][2] = fmaf(a4[u], __uint_as_float(bv[u].z), acc[m][2]);
                    acc[m][3] = fmaf(a4[u], __uint_as_float(bv[u].w), acc[m][3]);
                }
            }
        }
    }
    float* __restrict__ C = p.c + batch * p.sc + n0;
#pragma unroll
    for (int m = 0; m < MB; m++)
        if (m < p.M) *reinterpret_cast<float4*>(C + static_cast<int64_t>(m) * p.N) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
}

// The same walk for rows of B that are not 16-byte aligned (N % 4 != 0, e.g. a context length of 517): one
// thread per column, 4-byte loads of B that a warp coalesces into 128 contiguous bytes per k, sixteen k in
// flight per thread.  A still needs K % 4 == 0 and 16-byte alignment.
template <int MB>
__global__ void __launch_bounds__(256) smallk1_kernel(SkinnyParams p, int64_t total_cols, uint32_t n32) {
    dep_sync();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (idx >= total_cols) return;
    const int64_t batch = idx / n32;
    const int64_t n0 = idx - batch * n32;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb + n0;
    float acc[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) acc[m] = 0.f;
    const int K = static_cast<int>(p.K);
    int k = 0;
    for (; k + 16 <= K; k += 16) {
        float bv[16];
#pragma unroll
        for (int u = 0; u < 16; u++) bv[u] = __ldg(B + static_cast<int64_t>(k + u) * p.N);
#pragma unroll
        for (int m = 0; m < MB; m++) {
            if (m < p.M) {
#pragma unroll
                for (int q = 0; q < 4; q++) {
                    const float4 av = __ldg(reinterpret_cast<const float4*>(A + static_cast<int64_t>(m) * p.K + k + 4 * q));
                    acc[m] = fmaf(av.x, bv[4 * q + 0], acc[m]);
                    acc[m] = fmaf(av.y, bv[4 * q + 1], acc[m]);
                    acc[m] = fmaf(av.z, bv[4 * q + 2], acc[m]);
                    acc[m] = fmaf(av.w, bv[4 * q + 3], acc[m]);
                }
            }
        }
    }
    for (; k < K; k++) {
        const float b = __ldg(B + static_cast<int64_t>(k) * p.N);
#pragma unroll
        for (int m = 0; m < MB; m++)
            if (m < p.M) acc[m] = fmaf(__ldg(A + static_cast<int64_t>(m) * p.K + k), b, acc[m]);
    }
    float* __restrict__ C = p.c + batch * p.sc + n0;
#pragma unroll
    for (int m = 0; m < MB; m++)
        if (m < p.M) C[static_cast<int64_t>(m) * p.N] = acc[m];
}

// ---------------------------------------------------------------------------------------------
// C = A x B^T with B stored [N][K] row-major (what MatMul(A, Transpose(B)) computes, without the copy)
// ---------------------------------------------------------------------------------------------
// Few rows of A and a short K (decode attention scores against a [T, head_dim] key cache): a warp owns 32
// consecutive rows of B; LPR lanes share one row (each lane one 16-byte k-quad, so a warp-wide load reads
// 32 / LPR whole rows = 512 contiguous bytes), the k-quads of A live in registers, and the partial dot
// products are summed across the LPR lanes by shuffles.  For four rows of A the first two shuffle steps
// exchange halves of the four partial sums instead of all of them (5 shuffles per row instead of 16).
template <int MB, int LPR>
__global__ void __launch_bounds__(256) nt_rows_kernel(SkinnyParams p, uint32_t chunks_per_batch, int64_t total_chunks) {
    dep_sync();
    const int64_t wid = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    if (wid >= total_chunks) return;
    const int lane = threadIdx.x & 31;
    const int64_t batch = wid / chunks_per_batch;
    const int64_t n0 = (wid - batch * chunks_per_batch) * 32;
    constexpr int RPI = 32 / LPR;  // rows per warp-wide load
    const int sub = lane % LPR, rsel = lane / LPR;
    const bool kin = 4 * sub < p.K;
    float4 a[MB];
#pragma unroll
    for (int m = 0; m < MB; m++) {
        a[m] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kin && m < p.M) a[m] = __ldg(reinterpret_cast<const float4*>(p.a + batch * p.sa + static_cast<int64_t>(m) * p.K + 4 * sub));
    }
    const float* __restrict__ B = p.b + batch * p.sb + 4 * sub;
    float* __restrict__ C = p.c + batch * p.sc;
    constexpr int UN = LPR < 16 ? LPR : 16;  // a warp keeps up to 16 row loads (8 KB) in flight
    for (int it0 = 0; it0 < LPR; it0 += UN) {
        uint4 bv[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int64_t n = n0 + (it0 + u) * RPI + rsel;
            bv[u] = make_uint4(0, 0, 0, 0);
            if (kin && n < p.N) bv[u] = ld_stream_u4(B + n * p.K);
        }
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int64_t n = n0 + (it0 + u) * RPI + rsel;
            const float bx = __uint_as_float(bv[u].x), by = __uint_as_float(bv[u].y), bz = __uint_as_float(bv[u].z), bw = __uint_as_float(bv[u].w);
            float part[MB];
#pragma unroll
            for (int m = 0; m < MB; m++) part[m] = fmaf(a[m].w, bw, fmaf(a[m].z, bz, fmaf(a[m].y, by, a[m].x * bx)));
            if constexpr (MB == 4 && LPR >= 4) {
                const bool up1 = (sub & (LPR / 2)) != 0;
                const float r0 = __shfl_xor_sync(0xffffffffu, up1 ? part[0] : part[2], LPR / 2);
                const float r1 = __shfl_xor_sync(0xffffffffu, up1 ? part[1] : part[3], LPR / 2);
                const float q0 = (up1 ? part[2] : part[0]) + r0;
                const float q1 = (up1 ? part[3] : part[1]) + r1;
                const bool up2 = (sub & (LPR / 4)) != 0;
                const float r2 = __shfl_xor_sync(0xffffffffu, up2 ? q0 : q1, LPR / 4);
                float v = (up2 ? q1 : q0) + r2;
#pragma unroll
                for (int off = LPR / 8; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                const int m = 2 * (up1 ? 1 : 0) + (up2 ? 1 : 0);
                if ((sub & (LPR / 4 - 1)) == 0 && n < p.N && m < p.M) C[static_cast<int64_t>(m) * p.N + n] = v;
            } else {
#pragma unroll
                for (int m = 0; m < MB; m++) {
                    float v = part[m];
#pragma unroll
                    for (int off = LPR / 2; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
                    if (sub == 0 && n < p.N && m < p.M) C[static_cast<int64_t>(m) * p.N + n] = v;
                }
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------
// Few rows of A against a narrow B (N <= 128), many problems, any K: decode attention context
// ([4 heads, T] x [T, head_dim] per KV head).  One CTA per problem; LPR = N / 4 lanes cover one row of B (a
// warp-wide load reads 32 / LPR whole rows, contiguous in memory), the 8 warps take successive row groups, A is
// staged per k-chunk in shared memory as [k][m] so that one 16-byte shared load feeds the FMAs of four rows of A.
// The k-lanes are added at the end: inside a warp by shuffles, across warps through shared memory in warp order.
// ---------------------------------------------------------------------------------------------
constexpr int NN_KC = 512;  // k-chunk of A staged in shared memory

template <int MB, int LPR>
__global__ void __launch_bounds__(256) nn_narrow_kernel(SkinnyParams p) {
    dep_sync();
    constexpr int RPI = 32 / LPR;      // rows of B per warp-wide load
    constexpr int ROWS = 8 * RPI;      // rows of B per CTA-wide load
    constexpr int SA = MB < 4 ? MB : ((MB + 3) / 4) * 4;
    __shared__ __align__(16) float sA[NN_KC * SA];
    __shared__ __align__(16) float sRed[8 * MB * LPR * 4];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rsel = lane / LPR;
    const int64_t batch = blockIdx.x;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb + 4 * sub;
    const bool nin = 4 * sub < p.N;
    float acc[MB][4];
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;
    for (int64_t kc = 0; kc < p.K; kc += NN_KC) {
        const int kn = static_cast<int>(p.K - kc < NN_KC ? p.K - kc : NN_KC);
        __syncthreads();
        for (int i = threadIdx.x; i < NN_KC * MB; i += 256) {
            const int m = i / NN_KC, k = i - m * NN_KC;  // consecutive threads read consecutive k
            sA[k * SA + m] = (m < p.M && k < kn) ? A[static_cast<int64_t>(m) * p.K + kc + k] : 0.f;
        }
        __syncthreads();
        for (int k0 = warp * RPI + rsel; k0 < kn; k0 += 8 * ROWS) {
            uint4 bv[8];
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int k = k0 + u * ROWS;
                bv[u] = make_uint4(0, 0, 0, 0);
                if (nin && k < kn) bv[u] = ld_stream_u4(B + (kc + k) * p.N);
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                const int k = k0 + u * ROWS;
                if (k < kn) {
                    const float bx = __uint_as_float(bv[u].x), by = __uint_as_float(bv[u].y), bz = __uint_as_float(bv[u].z), bw = __uint_as_float(bv[u].w);
                    float av[SA];
                    if constexpr (SA % 4 == 0) {
#pragma unroll
                        for (int m = 0; m < SA; m += 4) {
                            const float4 t = *reinterpret_cast<const float4*>(sA + k * SA + m);
                            av[m] = t.x; av[m + 1] = t.y; av[m + 2] = t.z; av[m + 3] = t.w;
                        }
                    } else {
#pragma unroll
                        for (int m = 0; m < SA; m++) av[m] = sA[k * SA + m];
                    }
#pragma unroll
                    for (int m = 0; m < MB; m++) {
                        acc[m][0] = fmaf(av[m], bx, acc[m][0]);
                        acc[m][1] = fmaf(av[m], by, acc[m][1]);
                        acc[m][2] = fmaf(av[m], bz, acc[m][2]);
                        acc[m][3] = fmaf(av[m], bw, acc[m][3]);
                    }
                }
            }
        }
    }
    // add the row groups of a warp, then the 8 warps in order
#pragma unroll
    for (int m = 0; m < MB; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float v = acc[m][j];
#pragma unroll
            for (int off = LPR; off < 32; off <<= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
            acc[m][j] = v;
        }
    if (rsel == 0) {
#pragma unroll
        for (int m = 0; m < MB; m++)
            *reinterpret_cast<float4*>(sRed + ((warp * MB + m) * LPR + sub) * 4) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    }
    __syncthreads();
    float* __restrict__ C = p.c + batch * p.sc;
    for (int i = threadIdx.x; i < MB * LPR * 4; i += 256) {
        const int m = i / (LPR * 4), n = i - m * (LPR * 4);
        if (m < p.M && n < p.N) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) s += sRed[(w * MB + m) * LPR * 4 + n];
            C[static_cast<int64_t>(m) * p.N + n] = s;
        }
    }
}

// Any other shape: one thread per output element, sequential fp32 dot product.
__global__ void __launch_bounds__(256) nt_generic_kernel(SkinnyParams p, int64_t total) {
    dep_sync();
    const int64_t idx = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (idx >= total) return;
    const int64_t mn = p.M * p.N;
    const int64_t batch = idx / mn, r = idx - batch * mn;
    const int64_t m = r / p.N, n = r - m * p.N;
    const float* __restrict__ A = p.a + batch * p.sa + m * p.K;
    const float* __restrict__ B = p.b + batch * p.sb + n * p.K;
    float s = 0.f;
    for (int64_t k = 0; k < p.K; k++) s = fmaf(A[k], B[k], s);
    p.c[batch * p.sc + r] = s;
}

// Sum the split-K partials [ksplit][batch][M*N] in split order.
__global__ void __launch_bounds__(256) splitk_reduce_kernel(const float* __restrict__ part, float* __restrict__ c, int ksplit,
                                                            int64_t batch, int64_t mn, int64_t sc) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= batch * mn) return;
    const int64_t b = i / mn, e = i - b * mn;
    float s = 0.f;
    for (int k = 0; k < ksplit; k++) s += part[(static_cast<int64_t>(k) * batch + b) * mn + e];
    c[b * sc + e] = s;
}

// ---------------------------------------------------------------------------------------------
// tiled SIMT GEMM
// ---------------------------------------------------------------------------------------------
constexpr int GM_BK = 16;

struct GemmParams {
    const float* a;
    const float* b;
    float* c;
    int64_t M, N, K;
    int64_t sa, sb, sc;
    int vec_a, vec_b;  // rows of A / B are 16-byte aligned
};

template <int BM, int BN>
__global__ void __launch_bounds__(256) gemm_kernel(GemmParams p) {
    dep_sync();
    constexpr int TM = BM / 16, TN = BN / 16;
    __shared__ __align__(16) float As[2][GM_BK][BM + 4];
    __shared__ __align__(16) float Bs[2][GM_BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;
    const int64_t batch = blockIdx.z;
    const int64_t m0 = static_cast<int64_t>(blockIdx.y) * BM, n0 = static_cast<int64_t>(blockIdx.x) * BN;
    const float* __restrict__ A = p.a + batch * p.sa;
    const float* __restrict__ B = p.b + batch * p.sb;
    float* __restrict__ C = p.c + batch * p.sc;

    // loader mapping: A tile is BM x 16 (k contiguous): quads along k -> BM*4 quads; B tile is 16 x BN: BN/4 quads per row
    constexpr int A_QUADS = BM * GM_BK / 4, B_QUADS = BN * GM_BK / 4;
    constexpr int A_PER = (A_QUADS + 255) / 256, B_PER = (B_QUADS + 255) / 256;
    float4 ra[A_PER], rb[B_PER];

    auto load_tiles = [&](int64_t k0) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            const int q = tid + i * 256;
            ra[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (q < A_QUADS) {
                const int row = q >> 2, kq = (q & 3) * 4;
                const int64_t gm = m0 + row, gk = k0 + kq;
                if (gm < p.M) {
                    const float* src = A + gm * p.K + gk;
                    if (p.vec_a && gk + 3 < p.K) {
                        ra[i] = *reinterpret_cast<const float4*>(src);
                    } else {
                        if (gk + 0 < p.K) ra[i].x = src[0];
                        if (gk + 1 < p.K) ra[i].y = src[1];
                        if (gk + 2 < p.K) ra[i].z = src[2];
                        if (gk + 3 < p.K) ra[i].w = src[3];
                    }
                }
            }
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            const int q = tid + i * 256;
            rb[i] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (q < B_QUADS) {
                const int row = q / (BN / 4), cq = (q - row * (BN / 4)) * 4;
                const int64_t gk = k0 + row, gn = n0 + cq;
                if (gk < p.K) {
                    const float* src = B + gk * p.N + gn;
                    if (p.vec_b && gn + 3 < p.N) {
                        rb[i] = *reinterpret_cast<const float4*>(src);
                    } else {
                        if (gn + 0 < p.N) rb[i].x = src[0];
                        if (gn + 1 < p.N) rb[i].y = src[1];
                        if (gn + 2 < p.N) rb[i].z = src[2];
                        if (gn + 3 < p.N) rb[i].w = src[3];
                    }
                }
            }
        }
    };
    auto store_tiles = [&](int buf) {
#pragma unroll
        for (int i = 0; i < A_PER; i++) {
            const int q = tid + i * 256;
            if (q < A_QUADS) {
                const int row = q >> 2, kq = (q & 3) * 4;
                As[buf][kq + 0][row] = ra[i].x;
                As[buf][kq + 1][row] = ra[i].y;
                As[buf][kq + 2][row] = ra[i].z;
                As[buf][kq + 3][row] = ra[i].w;
            }
        }
#pragma unroll
        for (int i = 0; i < B_PER; i++) {
            const int q = tid + i * 256;
            if (q < B_QUADS) {
                const int row = q / (BN / 4), cq = (q - row * (BN / 4)) * 4;
                *reinterpret_cast<float4*>(&Bs[buf][row][cq]) = rb[i];
            }
        }
    };

    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    const int64_t nk = (p.K + GM_BK - 1) / GM_BK;
    load_tiles(0);
    store_tiles(0);
    __syncthreads();
    for (int64_t kt = 0; kt < nk; kt++) {
        const int buf = static_cast<int>(kt & 1);
        if (kt + 1 < nk) load_tiles((kt + 1) * GM_BK);
#pragma unroll
        for (int k = 0; k < GM_BK; k++) {
            float a[TM], b[TN];
            // thread (ty, tx) owns rows ty*4 + {0..3} (+64 for the second half when TM == 8) and the
            // matching column pattern: 4-wide pieces keep the shared-memory reads 128-bit and conflict-free
#pragma unroll
            for (int i = 0; i < TM; i += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&As[buf][k][ty * 4 + i * 16]);
                a[i] = v.x; a[i + 1] = v.y; a[i + 2] = v.z; a[i + 3] = v.w;
            }
#pragma unroll
            for (int j = 0; j < TN; j += 4) {
                const float4 v = *reinterpret_cast<const float4*>(&Bs[buf][k][tx * 4 + j * 16]);
                b[j] = v.x; b[j + 1] = v.y; b[j + 2] = v.z; b[j + 3] = v.w;
            }
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        if (kt + 1 < nk) {
            store_tiles(buf ^ 1);
            __syncthreads();
        }
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int64_t gm = m0 + ty * 4 + (i / 4) * 64 + (i % 4);
        if (gm >= p.M) continue;
#pragma unroll
        for (int j = 0; j < TN; j += 4) {
            const int64_t gn = n0 + tx * 4 + (j / 4) * 64;
            float* dst = C + gm * p.N + gn;
            if (p.vec_b && gn + 3 < p.N) {
                *reinterpret_cast<float4*>(dst) = make_float4(acc[i][j], acc[i][j + 1], acc[i][j + 2], acc[i][j + 3]);
            } else {
#pragma unroll
                for (int e = 0; e < 4; e++)
                    if (gn + e < p.N) dst[e] = acc[i][j + e];
            }
        }
    }
}

template <int MB>
static void skinny_launch(cudaStream_t st, const SkinnyParams& p, dim3 grid) {
    launch_dep(skinny_kernel<MB>, dim3(grid), dim3(SK_THREADS), 0, st, p);
}

static bool gemv_wide_enabled() {
    static const bool v = [] {
        const char* e = getenv("RMLK_B200_NO_GEMV_WIDE");
        return !(e && e[0] == '1');
    }();
    return v;
}

static int skinny_plan(int64_t batch, int64_t n, int64_t k) {
    // number of K splits that brings the grid to about two CTAs per SM
    const int64_t strips = ceil_div64(n, SK_COLS) * batch;
    const int64_t target = 2ll * sm_count();
    if (strips >= target) return 1;
    int64_t s = ceil_div64(target, strips);
    const int64_t max_s = ceil_div64(k, 2 * SK_KC);  // keep at least two chunks per split
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    return static_cast<int>(s > 64 ? 64 : s);
}

}  // namespace rmlk

using namespace rmlk;

namespace rmlk {
// tensor-core path (matmul_tc.cu)
bool tc_matmul_eligible(int64_t m, int64_t n, int64_t k, const void* a, const void* w, const void* c);
size_t tc_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k);
int tc_matmul(cudaStream_t st, int64_t m, int64_t n, int64_t k, const float* a, const float* w, float* c, void* workspace,
              size_t workspace_bytes, int* status, int* ksplit_out, int flags, int64_t ld, const TcPeers* peers = nullptr);
int tc_matmul_plan(int64_t m, int64_t n, int64_t k);
// fewest rows of A the tensor-core path takes: from 5 rows on, one pass of the weight-streaming tensor-core kernel (its 64-row
// tile mostly padding) beats the SIMT small-M kernels; up to 4 rows the wide-strip SIMT kernel is at the HBM stream's speed
constexpr int64_t TC_MIN_ROWS = 5;
bool tc_enabled();
// matmul_f16.cu
int matmul_f16(cudaStream_t st, int64_t batch, int64_t m, int64_t n, int64_t k, const void* a, int64_t sa, const void* b, int64_t sb, void* c,
               int64_t sc);
}  // namespace rmlk

extern "C" size_t rmlk_b200_matmul_workspace_bytes(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k) {
    if (dtype != RMLK_F32 || batch <= 0 || m <= 0 || n <= 0 || k <= 0) return 0;
    if (batch == 1 && m >= TC_MIN_ROWS && tc_enabled() && n % 128 == 0 && k % 32 == 0 && k >= 32) return tc_matmul_workspace_bytes(m, n, k);
    if (m > 16) return 0;
    const int s = skinny_plan(batch, n, k);
    size_t need = s > 1 ? static_cast<size_t>(s) * batch * m * n * sizeof(float) : 0;
    if (n % 4 == 0 && n >= GW_COLS && gemv_wide_enabled()) {  // the wide-strip kernel's split (taken when the operands are aligned)
        int64_t kps = k;
        const int sw = gemv_wide_plan(batch, m, n, k, &kps);
        const size_t need_w = sw > 1 ? static_cast<size_t>(sw) * batch * m * n * sizeof(float) : 0;
        if (need_w > need) need = need_w;
    }
    return need;
}

extern "C" int rmlk_b200_matmul(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                                const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                                int64_t c_batch_stride, void* workspace, size_t workspace_bytes) {
    return rmlk_b200_matmul_ex(stream, dtype, batch, m, n, k, a, a_batch_stride, b, b_batch_stride, c, c_batch_stride, workspace,
                               workspace_bytes, nullptr);
}

// dst[i] = 0.f + src[0][i] + src[1][i] + ... : the split-K reduction as an entry point of its own.
extern "C" int rmlk_b200_sum_parts(rmlk_stream_t stream, int dtype, int parts, int64_t n, const void* src, void* dst) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for sum_parts (f32 only)");
    if (parts < 1 || n < 0) return fail(RMLK_ERR_INVALID_ARG, "sum_parts: bad extent");
    if (n == 0) return RMLK_OK;
    if (!src || !dst) return fail(RMLK_ERR_INVALID_ARG, "sum_parts: NULL pointer");
    if (ceil_div64(n, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "sum_parts: tensor too large");
    launch_dep(splitk_reduce_kernel, dim3(static_cast<unsigned>(ceil_div64(n, 256))), dim3(256), 0, as_stream(stream), static_cast<const float*>(src),
                                                                                                  static_cast<float*>(dst), parts, 1, n, n);
    RMLK_CHECK_LAUNCH("splitk_reduce_kernel");
    return RMLK_OK;
}

// C[:, 0:n] = A x B[:, 0:n] where b and c point at the first column of a block of n columns inside matrices whose rows are
// ld elements apart: lets a wide product (the logits of a language model) be issued block by block, so that what
// follows a block - a copy to the host - overlaps the next.  Only shapes the tensor-core kernel runs without a K split.
extern "C" int rmlk_b200_matmul_window_supported(int64_t m, int64_t n, int64_t k, int64_t ld) {
    return tc_enabled() && m >= TC_MIN_ROWS && n > 0 && n % 128 == 0 && k >= 32 && k % 32 == 0 && ld >= n && ld % 4 == 0 && tc_matmul_plan(m, n, k) == 1;
}

extern "C" int rmlk_b200_matmul_window(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, const void* b, void* c,
                                       int64_t ld, int* status, int flags) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for matmul_window (f32 only)");
    if (!a || !b || !c) return fail(RMLK_ERR_INVALID_ARG, "matmul_window: NULL operand");
    if (!rmlk_b200_matmul_window_supported(m, n, k, ld) || !tc_matmul_eligible(m, n, k, a, b, c))
        return fail(RMLK_ERR_INVALID_ARG, "matmul_window: needs M >= 5, N % 128 == 0, K % 32 == 0, 16-byte aligned operands and a shape without a K split");
    int ksplit = 1;
    return tc_matmul(as_stream(stream), m, n, k, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c), nullptr, 0,
                     status, &ksplit, flags, ld);
}

// C[m,n] = A x B for a caller that adds the split-K partial sums itself (in its next kernel): when the plan for this
// shape splits K through the workspace, the slabs are left there ([*parts][m*n] floats, to be added in slab order
// starting from 0.f) and C is not written; otherwise C is complete and *parts = 1.
extern "C" int rmlk_b200_matmul_parts(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, const void* b, void* c,
                                      void* workspace, size_t workspace_bytes, int* status, int flags, int* parts) {
    if (!parts) return fail(RMLK_ERR_INVALID_ARG, "matmul_parts: NULL parts");
    *parts = 1;
    if (dtype == RMLK_F32 && m > 0 && n > 0 && k > 0 && a && b && c && tc_matmul_eligible(m, n, k, a, b, c)) {
        int ksplit = 1;
        if (int rc = tc_matmul(as_stream(stream), m, n, k, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c),
                               workspace, workspace_bytes, status, &ksplit, flags, 0))
            return rc;
        *parts = ksplit;
        return RMLK_OK;
    }
    return rmlk_b200_matmul_flags(stream, dtype, 1, m, n, k, a, 0, b, 0, c, 0, workspace, workspace_bytes, status, flags);
}

extern "C" int rmlk_b200_matmul_ex(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                                   const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                                   int64_t c_batch_stride, void* workspace, size_t workspace_bytes, int* status) {
    return rmlk_b200_matmul_flags(stream, dtype, batch, m, n, k, a, a_batch_stride, b, b_batch_stride, c, c_batch_stride, workspace,
                                  workspace_bytes, status, 0);
}

extern "C" int rmlk_b200_matmul_flags(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                                      const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                                      int64_t c_batch_stride, void* workspace, size_t workspace_bytes, int* status, int flags) {
    if (dtype == RMLK_F16) {
        if (batch < 0 || m < 0 || n < 0 || k < 0) return fail(RMLK_ERR_INVALID_ARG, "matmul: negative extent");
        if (batch == 0 || m == 0 || n == 0) return RMLK_OK;
        if (!c || (k > 0 && (!a || !b))) return fail(RMLK_ERR_INVALID_ARG, "matmul: NULL operand");
        return matmul_f16(as_stream(stream), batch, m, n, k, a, a_batch_stride, b, b_batch_stride, c, c_batch_stride);
    }
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for matmul (f32 and f16)");
    if (batch < 0 || m < 0 || n < 0 || k < 0) return fail(RMLK_ERR_INVALID_ARG, "matmul: negative extent");
    if (batch == 0 || m == 0 || n == 0) return RMLK_OK;
    if (!c) return fail(RMLK_ERR_INVALID_ARG, "matmul: NULL output");
    cudaStream_t st = as_stream(stream);
    if (k == 0) {  // empty sum: C = 0
        for (int64_t bi = 0; bi < batch; bi++)
            RMLK_CUDA(cudaMemsetAsync(static_cast<float*>(c) + bi * c_batch_stride, 0, static_cast<size_t>(m) * n * sizeof(float), st));
        return RMLK_OK;
    }
    if (!a || !b) return fail(RMLK_ERR_INVALID_ARG, "matmul: NULL operand");
    if (batch > 65535) return fail(RMLK_ERR_INVALID_ARG, "matmul: batch exceeds 65535");
    const bool b_rows_aligned = (n % 4 == 0) && aligned_to(b, 16) && (b_batch_stride % 4 == 0);
    if (batch == 1 && tc_matmul_eligible(m, n, k, a, b, c)) {
        int ksplit = 1;
        if (int rc = tc_matmul(st, m, n, k, static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(c), workspace,
                               workspace_bytes, status, &ksplit, flags, 0))
            return rc;
        if (ksplit > 1) {
            const int64_t total = m * n;
            launch_dep(splitk_reduce_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, st, static_cast<const float*>(workspace),
                                                                                                  static_cast<float*>(c), ksplit, 1, total, total);
            RMLK_CHECK_LAUNCH("splitk_reduce_kernel");
        }
        return RMLK_OK;
    }
    if (m <= 16) {
        SkinnyParams p;
        p.a = static_cast<const float*>(a);
        p.b = static_cast<const float*>(b);
        p.M = m; p.N = n; p.K = k;
        p.sa = a_batch_stride; p.sb = b_batch_stride; p.sc = c_batch_stride;
        p.vec_b = b_rows_aligned ? 1 : 0;
        // many problems with a short K: one thread per column quad (or per column), no reduction
        if (m <= 4 && k <= 256 && k % 4 == 0 && aligned_to(a, 16) && a_batch_stride % 4 == 0 && n <= 0x7fffffffll &&
            batch * n >= 2048ll * sm_count() && batch * n < (1ll << 38)) {
            p.ksplit = 1;
            p.k_per_split = k;
            p.c = static_cast<float*>(c);
            if (b_rows_aligned && aligned_to(c, 16) && c_batch_stride % 4 == 0) {
                const int64_t total_quads = batch * (n / 4);
                const unsigned grid = static_cast<unsigned>(ceil_div64(total_quads, 256));
                if (m == 1) launch_dep(smallk_kernel<1>, dim3(grid), dim3(256), 0, st, p, total_quads, static_cast<uint32_t>(n / 4));
                else if (m == 2) launch_dep(smallk_kernel<2>, dim3(grid), dim3(256), 0, st, p, total_quads, static_cast<uint32_t>(n / 4));
                else launch_dep(smallk_kernel<4>, dim3(grid), dim3(256), 0, st, p, total_quads, static_cast<uint32_t>(n / 4));
            } else {
                const int64_t total_cols = batch * n;
                const unsigned grid = static_cast<unsigned>(ceil_div64(total_cols, 256));
                if (m == 1) launch_dep(smallk1_kernel<1>, dim3(grid), dim3(256), 0, st, p, total_cols, static_cast<uint32_t>(n));
                else if (m == 2) launch_dep(smallk1_kernel<2>, dim3(grid), dim3(256), 0, st, p, total_cols, static_cast<uint32_t>(n));
                else launch_dep(smallk1_kernel<4>, dim3(grid), dim3(256), 0, st, p, total_cols, static_cast<uint32_t>(n));
            }
            RMLK_CHECK_LAUNCH("smallk_kernel");
            return RMLK_OK;
        }
        // many problems with a narrow B: one CTA per problem reading whole rows of B
        if (m <= 4 && n <= 128 && b_rows_aligned && batch >= sm_count() && batch <= 0x7fffffffll) {
            p.ksplit = 1;
            p.k_per_split = k;
            p.c = static_cast<float*>(c);
            const unsigned grid = static_cast<unsigned>(batch);
#define RMLK_NN_NARROW(MB)                                                            \
    if (n <= 32) launch_dep(nn_narrow_kernel<MB, 8>, dim3(grid), dim3(256), 0, st, p);                    \
    else if (n <= 64) launch_dep(nn_narrow_kernel<MB, 16>, dim3(grid), dim3(256), 0, st, p);              \
    else launch_dep(nn_narrow_kernel<MB, 32>, dim3(grid), dim3(256), 0, st, p);
            if (m == 1) { RMLK_NN_NARROW(1) }
            else if (m == 2) { RMLK_NN_NARROW(2) }
            else { RMLK_NN_NARROW(4) }
#undef RMLK_NN_NARROW
            RMLK_CHECK_LAUNCH("nn_narrow_kernel");
            return RMLK_OK;
        }
        if (b_rows_aligned && aligned_to(c, 16) && c_batch_stride % 4 == 0 && n >= GW_COLS && gemv_wide_enabled()) {
            int64_t kps = k;
            int ksplit = gemv_wide_plan(batch, m, n, k, &kps);
            const size_t need = static_cast<size_t>(ksplit) * batch * m * n * sizeof(float);
            if (ksplit > 1 && (!workspace || workspace_bytes < need || !aligned_to(workspace, 16))) {
                ksplit = 1;
                kps = k;
            }
            p.ksplit = ksplit;
            p.k_per_split = kps;
            p.c = ksplit > 1 ? static_cast<float*>(workspace) : static_cast<float*>(c);
            dim3 grid(static_cast<unsigned>(ceil_div64(n, GW_COLS)), ksplit, static_cast<unsigned>(batch));
            if (m == 1) launch_dep(gemv_wide_kernel<1>, grid, dim3(GW_THREADS), 0, st, p);
            else if (m == 2) launch_dep(gemv_wide_kernel<2>, grid, dim3(GW_THREADS), 0, st, p);
            else if (m <= 4) launch_dep(gemv_wide_kernel<4>, grid, dim3(GW_THREADS), 0, st, p);
            else if (m <= 8) launch_dep(gemv_wide_kernel<8>, grid, dim3(GW_THREADS), 0, st, p);
            else launch_dep(gemv_wide_kernel<16>, grid, dim3(GW_THREADS), 0, st, p);
            RMLK_CHECK_LAUNCH("gemv_wide_kernel");
            if (ksplit > 1) {
                const int64_t total = batch * m * n;
                launch_dep(splitk_reduce_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, st,
                           static_cast<const float*>(workspace), static_cast<float*>(c), ksplit, batch, m * n, c_batch_stride);
                RMLK_CHECK_LAUNCH("splitk_reduce_kernel");
            }
            return RMLK_OK;
        }
        int ksplit = skinny_plan(batch, n, k);
        const size_t need = static_cast<size_t>(ksplit) * batch * m * n * sizeof(float);
        if (ksplit > 1 && (!workspace || workspace_bytes < need)) ksplit = 1;
        p.ksplit = ksplit;
        p.k_per_split = ksplit > 1 ? ceil_div64(ceil_div64(k, ksplit), SK_KC) * SK_KC : k;
        if (ksplit > 1) p.ksplit = ksplit = static_cast<int>(ceil_div64(k, p.k_per_split));
        p.c = ksplit > 1 ? static_cast<float*>(workspace) : static_cast<float*>(c);
        dim3 grid(static_cast<unsigned>(ceil_div64(n, SK_COLS)), ksplit, static_cast<unsigned>(batch));
        if (m == 1) skinny_launch<1>(st, p, grid);
        else if (m == 2) skinny_launch<2>(st, p, grid);
        else if (m <= 4) skinny_launch<4>(st, p, grid);
        else if (m <= 8) skinny_launch<8>(st, p, grid);
        else skinny_launch<16>(st, p, grid);
        RMLK_CHECK_LAUNCH("skinny_kernel");
        if (ksplit > 1) {
            const int64_t total = batch * m * n;
            launch_dep(splitk_reduce_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, st, 
                static_cast<const float*>(workspace), static_cast<float*>(c), ksplit, batch, m * n, c_batch_stride);
            RMLK_CHECK_LAUNCH("splitk_reduce_kernel");
        }
        return RMLK_OK;
    }
    GemmParams g;
    g.a = static_cast<const float*>(a);
    g.b = static_cast<const float*>(b);
    g.c = static_cast<float*>(c);
    g.M = m; g.N = n; g.K = k;
    g.sa = a_batch_stride; g.sb = b_batch_stride; g.sc = c_batch_stride;
    g.vec_a = ((k % 4 == 0) && aligned_to(a, 16) && (a_batch_stride % 4 == 0)) ? 1 : 0;
    g.vec_b = (b_rows_aligned && aligned_to(c, 16) && (c_batch_stride % 4 == 0)) ? 1 : 0;
    const int64_t tiles128 = ceil_div64(m, 128) * ceil_div64(n, 128) * batch;
    if (m > 64 && tiles128 >= sm_count()) {
        dim3 grid(static_cast<unsigned>(ceil_div64(n, 128)), static_cast<unsigned>(ceil_div64(m, 128)), static_cast<unsigned>(batch));
        launch_dep(gemm_kernel<128, 128>, dim3(grid), dim3(256), 0, st, g);
    } else {
        dim3 grid(static_cast<unsigned>(ceil_div64(n, 64)), static_cast<unsigned>(ceil_div64(m, 64)), static_cast<unsigned>(batch));
        launch_dep(gemm_kernel<64, 64>, dim3(grid), dim3(256), 0, st, g);
    }
    RMLK_CHECK_LAUNCH("gemm_kernel");
    return RMLK_OK;
}

template <int MB>
static void nt_rows_launch(cudaStream_t st, const SkinnyParams& p, int64_t batch) {
    const int64_t chunks = ceil_div64(p.N, 32);
    const int64_t total = chunks * batch;
    const unsigned grid = static_cast<unsigned>(ceil_div64(total, 8));
    if (p.K <= 16) launch_dep(nt_rows_kernel<MB, 4>, dim3(grid), dim3(256), 0, st, p, static_cast<uint32_t>(chunks), total);
    else if (p.K <= 32) launch_dep(nt_rows_kernel<MB, 8>, dim3(grid), dim3(256), 0, st, p, static_cast<uint32_t>(chunks), total);
    else if (p.K <= 64) launch_dep(nt_rows_kernel<MB, 16>, dim3(grid), dim3(256), 0, st, p, static_cast<uint32_t>(chunks), total);
    else launch_dep(nt_rows_kernel<MB, 32>, dim3(grid), dim3(256), 0, st, p, static_cast<uint32_t>(chunks), total);
}

extern "C" int rmlk_b200_matmul_nt(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k, const void* a,
                                   int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c, int64_t c_batch_stride) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for matmul (f32 only)");
    if (batch < 0 || m < 0 || n < 0 || k < 0) return fail(RMLK_ERR_INVALID_ARG, "matmul_nt: negative extent");
    if (batch == 0 || m == 0 || n == 0) return RMLK_OK;
    if (!c) return fail(RMLK_ERR_INVALID_ARG, "matmul_nt: NULL output");
    cudaStream_t st = as_stream(stream);
    if (k == 0) {
        for (int64_t bi = 0; bi < batch; bi++)
            RMLK_CUDA(cudaMemsetAsync(static_cast<float*>(c) + bi * c_batch_stride, 0, static_cast<size_t>(m) * n * sizeof(float), st));
        return RMLK_OK;
    }
    if (!a || !b) return fail(RMLK_ERR_INVALID_ARG, "matmul_nt: NULL operand");
    SkinnyParams p;
    p.a = static_cast<const float*>(a);
    p.b = static_cast<const float*>(b);
    p.c = static_cast<float*>(c);
    p.M = m; p.N = n; p.K = k;
    p.sa = a_batch_stride; p.sb = b_batch_stride; p.sc = c_batch_stride;
    p.k_per_split = k;
    p.vec_b = 1;
    const int64_t chunks = ceil_div64(n, 32) * batch;
    if (m <= 8 && k <= 128 && k % 4 == 0 && aligned_to(a, 16) && aligned_to(b, 16) && a_batch_stride % 4 == 0 && b_batch_stride % 4 == 0 &&
        batch <= 0x7fffffffll && chunks / 8 < 0x7fffffffll) {
        p.ksplit = 1;
        if (m == 1) nt_rows_launch<1>(st, p, batch);
        else if (m == 2) nt_rows_launch<2>(st, p, batch);
        else if (m <= 4) nt_rows_launch<4>(st, p, batch);
        else nt_rows_launch<8>(st, p, batch);
        RMLK_CHECK_LAUNCH("nt_rows_kernel");
        return RMLK_OK;
    }
    const int64_t total = batch * m * n;
    if (total / 256 >= 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "matmul_nt: output too large");
    p.ksplit = 1;
    launch_dep(nt_generic_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, st, p, total);
    RMLK_CHECK_LAUNCH("nt_generic_kernel");
    return RMLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Gemm epilogue: y = alpha * y + beta * c, c broadcast to [m, n] by strides (0 = broadcast)
// ---------------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(256) scale_add_bias_kernel(T* __restrict__ y, const T* __restrict__ c, int64_t total, uint32_t n, FastDiv ndiv,
                                                             int64_t cs_row, int64_t cs_col, float alpha, float beta) {
    dep_sync();
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
        float v = static_cast<float>(y[i]);
        if (alpha != 1.f) v = __fmul_rn(alpha, v);
        if (c) {
            uint32_t row, col;
            ndiv.divmod(static_cast<uint32_t>(i), row, col);
            v = fmaf(beta, static_cast<float>(c[row * cs_row + col * cs_col]), v);
        }
        y[i] = static_cast<T>(v);
    }
}

extern "C" int rmlk_b200_scale_add_bias(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, void* y, float alpha, const void* c,
                                        int64_t c_row_stride, int64_t c_col_stride, float beta) {
    if (dtype != RMLK_F32 && dtype != RMLK_F16) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for scale_add_bias (f32 and f16)");
    if (m < 0 || n < 0) return fail(RMLK_ERR_INVALID_ARG, "scale_add_bias: negative extent");
    if (m == 0 || n == 0 || (alpha == 1.f && !c)) return RMLK_OK;
    if (!y) return fail(RMLK_ERR_INVALID_ARG, "scale_add_bias: NULL output");
    if (m * n > 0x7fffffffll || n > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "scale_add_bias: more than 2^31 elements");
    const int64_t total = m * n;
    const unsigned grid = flat_grid(total, 256, 8);
    if (dtype == RMLK_F32)
        launch_dep(scale_add_bias_kernel<float>, dim3(grid), dim3(256), 0, as_stream(stream), static_cast<float*>(y), static_cast<const float*>(c), total,
                   static_cast<uint32_t>(n), FastDiv(static_cast<uint32_t>(n)), c_row_stride, c_col_stride, alpha, beta);
    else
        launch_dep(scale_add_bias_kernel<__half>, dim3(grid), dim3(256), 0, as_stream(stream), static_cast<__half*>(y), static_cast<const __half*>(c), total,
                   static_cast<uint32_t>(n), FastDiv(static_cast<uint32_t>(n)), c_row_stride, c_col_stride, alpha, beta);
    RMLK_CHECK_LAUNCH("scale_add_bias_kernel");
    return RMLK_OK;
}

// ---------------------------------------------------------------------------------------------
// MatMul without any allocation by anyone: the split-K scratch is a fixed array inside the library.
// ---------------------------------------------------------------------------------------------
// 8 MiB of device memory per GPU that loads this library, held until the process exits.
constexpr size_t RMLK_STATIC_SCRATCH_BYTES = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_matmul_static_scratch[RMLK_STATIC_SCRATCH_BYTES];

// In host code `g_matmul_static_scratch` is only a handle for the runtime, not a device address, so the
// address kernels can use is looked up once per device (with that device current) and cached.
static void* static_scratch_ptr(int* rc_out) {
    // One slot per device.  Threads that race on a device's first call all look the same address up and store the same
    // value; the atomic makes the publication well defined.
    static std::atomic<void*> ptrs[64];
    *rc_out = RMLK_OK;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) {
        *rc_out = rmlk::cuda_fail(e, "cudaGetDevice");
        return nullptr;
    }
    if (dev < 0 || dev >= 64) {
        *rc_out = rmlk::fail(RMLK_ERR_INTERNAL, "matmul_static: device index out of range");
        return nullptr;
    }
    void* p = ptrs[dev].load(std::memory_order_acquire);
    if (!p) {
        e = cudaGetSymbolAddress(&p, g_matmul_static_scratch);
        if (e != cudaSuccess || !p) {
            *rc_out = rmlk::cuda_fail(e, "cudaGetSymbolAddress(matmul static scratch)");
            return nullptr;
        }
        ptrs[dev].store(p, std::memory_order_release);
    }
    return p;
}

extern "C" size_t rmlk_b200_matmul_static_scratch_bytes(void) { return RMLK_STATIC_SCRATCH_BYTES; }

static size_t matmul_least_scratch(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k) {
    return rmlk_b200_matmul_workspace_bytes(dtype, batch, m, n, k);
}

extern "C" int rmlk_b200_matmul_static_supported(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k) {
    return matmul_least_scratch(dtype, batch, m, n, k) <= RMLK_STATIC_SCRATCH_BYTES ? 1 : 0;
}

extern "C" int rmlk_b200_matmul_static(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                                       const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                                       int64_t c_batch_stride, int* status) {
    const size_t need = matmul_least_scratch(dtype, batch, m, n, k);
    if (need > RMLK_STATIC_SCRATCH_BYTES)
        return rmlk::fail(RMLK_ERR_INVALID_ARG, "matmul_static: this shape needs " + std::to_string(need) +
                                                    " bytes of split-K scratch, the built-in array holds " +
                                                    std::to_string(RMLK_STATIC_SCRATCH_BYTES) +
                                                    "; use rmlk_b200_matmul with a caller-provided workspace");
    int rc = RMLK_OK;
    void* scratch = static_scratch_ptr(&rc);
    if (!scratch) return rc;
    // The split-K partials are fully overwritten before they are summed, so nothing in the array has to be
    // cleared between calls.
    return rmlk_b200_matmul_ex(stream, dtype, batch, m, n, k, a, a_batch_stride, b, b_batch_stride, c, c_batch_stride, scratch,
                               RMLK_STATIC_SCRATCH_BYTES, status);
}
