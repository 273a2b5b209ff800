// Decode attention over a KV cache read in place, one launch.  For every problem p (batch entry x KV head) and each
// of its R <= 4 query rows (the query heads that share the KV head, one new token each):
//     s[r][t] = (q[p][r] . K[p][t]) * scale + mask[b][h][t]      t < T keys
//     P[r][:] = softmax(s[r][:])
//     out[p][r] = sum_t P[r][t] * V[p][t]
// which an exported decoder graph spells MatMul(q, Transpose(K)) -> Mul -> Add -> Softmax -> MatMul(., V), with K and V
// first repeated per query head (Expand) and K transposed; the reference runs every one of those nodes as a launch
// with a copy of its own (backend/matmul.rs:223-356, mul.rs, add.rs, softmax.rs, expand.rs, transpose.rs).  Here K
// and V are read once, from the cache as it lies ([T, D] rows per problem, problems a fixed stride apart), and the
// scores never leave shared memory.
//
// One CTA of 8 warps per problem.  LPR = D / 4 lanes cover a row of K or V with one 16-byte load each, so a warp-wide
// load reads 32 / LPR whole rows (512 contiguous bytes); every warp keeps 16 such loads in flight.  The arithmetic
// follows the single kernels it stands for: dot products as in the A x B^T kernel (same FMA order, same shuffle
// butterfly), scale / mask / max / exp / sum / divide as in the softmax kernel (same expressions, same order), so
// the probabilities equal theirs bit for bit; the P x V sums associate differently from the stand-alone MatMul
// (within its 1e-4 bar).
//
// Measured on 512 problems x 4 rows x 550 keys x 64 (one layer of the decode benchmark), as the difference it makes
// to the 16-layer step: the one-CTA-per-problem kernel is about 15 us per layer slower than the A x B^T, softmax and
// narrow-MatMul kernels run one after the other (37 us), the split-keys kernel below about 6 us slower.  The host
// runtime therefore uses them only on request (RMLK_B200_ATTENTION=1).
#include <cstdlib>
#include <mutex>
#include "common.cuh"

namespace rmlk {

struct AttnParams {
    const float* q;
    const float* k;
    const float* v;
    const float* mask;  // may be null
    float* out;
    int64_t kb, vb;            // problem strides of K and V (elements)
    int64_t ms_b, ms_h;        // mask strides per batch entry and per head (elements; rows of T are dense)
    int rows, T, kv_heads;
    float scale;
};

template <int LPR>
__global__ void __launch_bounds__(256, 2) gqa_decode_attention_kernel(AttnParams p) {
    dep_sync();
    constexpr int D = 4 * LPR;
    constexpr int RPI = 32 / LPR;  // rows of K / V per warp-wide load
    constexpr int UN = 16;         // loads in flight per warp
    extern __shared__ __align__(16) float smem[];
    float* s = smem;                                    // [T][4]: scores, then probabilities, of the 4 query rows
    float* red = smem + 4 * ((p.T + 3) & ~3);           // [8 warps][4 rows][D]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rsel = lane / LPR;
    const int64_t prob = blockIdx.x;
    const int T = p.T;

    // ---- scores ----
    float4 a[4];
#pragma unroll
    for (int m = 0; m < 4; m++) {
        a[m] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < p.rows) a[m] = __ldg(reinterpret_cast<const float4*>(p.q + (prob * p.rows + m) * D + 4 * sub));
    }
    const int64_t b = prob / p.kv_heads, h0 = (prob % p.kv_heads) * p.rows;
    const float* __restrict__ K = p.k + prob * p.kb + 4 * sub;
    for (int t0 = 0; t0 < T; t0 += 8 * RPI * UN) {
        uint4 bv[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int t = t0 + (u * 8 + warp) * RPI + rsel;
            bv[u] = make_uint4(0, 0, 0, 0);
            if (t < T) bv[u] = ld_stream_u4(K + static_cast<int64_t>(t) * D);
        }
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int t = t0 + (u * 8 + warp) * RPI + rsel;
            const float bx = __uint_as_float(bv[u].x), by = __uint_as_float(bv[u].y), bz = __uint_as_float(bv[u].z), bw = __uint_as_float(bv[u].w);
            float part[4];
#pragma unroll
            for (int m = 0; m < 4; m++) part[m] = fmaf(a[m].w, bw, fmaf(a[m].z, bz, fmaf(a[m].y, by, a[m].x * bx)));
            // the four partial sums are added across the LPR lanes of the row; the first two steps exchange halves
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
            if ((sub & (LPR / 4 - 1)) == 0 && t < T && m < p.rows) {
                float x = __fmul_rn(v, p.scale);
                if (p.mask) x = __fadd_rn(x, p.mask[b * p.ms_b + (h0 + m) * p.ms_h + t]);
                s[4 * t + m] = x;
            }
        }
    }
    __syncthreads();

    // ---- softmax: warp m takes query row m ----
    if (warp < p.rows) {
        float mx = -INFINITY;
        for (int t = lane; t < T; t += 32) mx = fmaxf(mx, s[4 * t + warp]);
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int t = lane; t < T; t += 32) {
            const float e = expf(s[4 * t + warp] - mx);
            s[4 * t + warp] = e;
            sum += e;
        }
#pragma unroll
        for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        for (int t = lane; t < T; t += 32) s[4 * t + warp] = s[4 * t + warp] / sum;
    } else if (warp < 4) {
        for (int t = lane; t < T; t += 32) s[4 * t + warp] = 0.f;  // rows that do not exist contribute nothing below
    }
    __syncthreads();

    // ---- context ----
    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;
    const float* __restrict__ V = p.v + prob * p.vb + 4 * sub;
    for (int t0 = 0; t0 < T; t0 += 8 * RPI * UN) {
        uint4 bv[UN];
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int t = t0 + (u * 8 + warp) * RPI + rsel;
            bv[u] = make_uint4(0, 0, 0, 0);
            if (t < T) bv[u] = ld_stream_u4(V + static_cast<int64_t>(t) * D);
        }
#pragma unroll
        for (int u = 0; u < UN; u++) {
            const int t = t0 + (u * 8 + warp) * RPI + rsel;
            if (t < T) {
                const float4 pr = *reinterpret_cast<const float4*>(s + 4 * t);
                const float vx = __uint_as_float(bv[u].x), vy = __uint_as_float(bv[u].y), vz = __uint_as_float(bv[u].z), vw = __uint_as_float(bv[u].w);
                const float pm[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
                for (int m = 0; m < 4; m++) {
                    acc[m][0] = fmaf(pm[m], vx, acc[m][0]);
                    acc[m][1] = fmaf(pm[m], vy, acc[m][1]);
                    acc[m][2] = fmaf(pm[m], vz, acc[m][2]);
                    acc[m][3] = fmaf(pm[m], vw, acc[m][3]);
                }
            }
        }
    }
    // rows handled by the other lane groups of the warp, then the 8 warps in warp order
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float x = acc[m][j];
#pragma unroll
            for (int off = LPR; off < 32; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            acc[m][j] = x;
        }
    if (rsel == 0) {
#pragma unroll
        for (int m = 0; m < 4; m++)
            *reinterpret_cast<float4*>(red + (warp * 4 + m) * D + 4 * sub) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < p.rows * D; i += 256) {
        const int m = i / D, d = i - m * D;
        float x = 0.f;
#pragma unroll
        for (int w = 0; w < 8; w++) x += red[(w * 4 + m) * D + d];
        p.out[(prob * p.rows + m) * D + d] = x;
    }
}

// The same computation with the keys of a problem split over several CTAs (128 keys each, 32 per warp): many small
// CTAs keep far more loads in flight than one CTA per problem.  Every warp makes the softmax of its own 32 keys
// (local maximum m, e = exp(s - m), l = sum e, a = sum e * V), the four warps of a CTA and then the CTAs of a problem
// are merged by the usual rescaling (M = max m; L = sum l exp(m - M); A = sum a exp(m - M); out = A / L).  Partial
// results go through a scratch buffer; the CTA that arrives last for a problem (a counter per problem, left at zero
// again) merges them, in split order, so the result does not depend on timing.
constexpr int SPLIT_KEYS = 128;

struct AttnSplitParams {
    AttnParams base;
    int nsplit;
    int* counters;   // [problems], zero on entry and on exit
    float* partial;  // [problems][nsplit][8 + 4 * D]: M[4], L[4], A[4][D]
};

template <int LPR>
__global__ void __launch_bounds__(128) gqa_decode_attention_split_kernel(AttnSplitParams sp) {
    dep_sync();
    const AttnParams& p = sp.base;
    constexpr int D = 4 * LPR;
    constexpr int RPI = 32 / LPR;   // rows of K / V per warp-wide load
    constexpr int UN = 32 / RPI;    // loads per warp: 32 keys
    constexpr int REC = 8 + 4 * D;  // floats per partial record
    __shared__ __align__(16) float s_e[4][32][4];     // per warp: exp(score - local max) of its 32 keys, 4 rows
    __shared__ float s_m[4][4], s_l[4][4];            // per warp: local max, local sum per row
    __shared__ __align__(16) float s_a[4][4][D];      // per warp: sum e * V per row
    __shared__ int s_last;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rsel = lane / LPR;
    const int64_t prob = blockIdx.y;
    const int split = blockIdx.x;
    const int T = p.T;
    const int tw = split * SPLIT_KEYS + warp * 32;  // first key of this warp

    float4 a[4];
#pragma unroll
    for (int m = 0; m < 4; m++) {
        a[m] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (m < p.rows) a[m] = __ldg(reinterpret_cast<const float4*>(p.q + (prob * p.rows + m) * D + 4 * sub));
    }
    const int64_t b = prob / p.kv_heads, h0 = (prob % p.kv_heads) * p.rows;
    const float* __restrict__ K = p.k + prob * p.kb + 4 * sub;
    const float* __restrict__ V = p.v + prob * p.vb + 4 * sub;
    uint4 bv[UN];
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const int t = tw + u * RPI + rsel;
        bv[u] = make_uint4(0, 0, 0, 0);
        if (t < T) bv[u] = ld_stream_u4(K + static_cast<int64_t>(t) * D);
    }
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const int t = tw + u * RPI + rsel;
        const float bx = __uint_as_float(bv[u].x), by = __uint_as_float(bv[u].y), bz = __uint_as_float(bv[u].z), bw = __uint_as_float(bv[u].w);
        float part[4];
#pragma unroll
        for (int m = 0; m < 4; m++) part[m] = fmaf(a[m].w, bw, fmaf(a[m].z, bz, fmaf(a[m].y, by, a[m].x * bx)));
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
        if ((sub & (LPR / 4 - 1)) == 0) {
            float x = -INFINITY;  // keys beyond the end and rows that do not exist
            if (t < T && m < p.rows) {
                x = __fmul_rn(v, p.scale);
                if (p.mask) x = __fadd_rn(x, p.mask[b * p.ms_b + (h0 + m) * p.ms_h + t]);
            }
            s_e[warp][u * RPI + rsel][m] = x;
        }
    }
    // the values for the second pass are requested now; the softmax of the 32 keys runs while they are on their way
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const int t = tw + u * RPI + rsel;
        bv[u] = make_uint4(0, 0, 0, 0);
        if (t < T) bv[u] = ld_stream_u4(V + static_cast<int64_t>(t) * D);
    }
    __syncwarp();
    {
        // lane = key; the four rows one after the other
        const float4 sc = *reinterpret_cast<const float4*>(&s_e[warp][lane][0]);
        const float sv[4] = {sc.x, sc.y, sc.z, sc.w};
        float ev[4];
#pragma unroll
        for (int m = 0; m < 4; m++) {
            float mx = sv[m];
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
            const float e = mx == -INFINITY ? 0.f : expf(sv[m] - mx);
            float sum = e;
#pragma unroll
            for (int o = 16; o >= 1; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
            ev[m] = e;
            if (lane == 0) {
                s_m[warp][m] = mx;
                s_l[warp][m] = sum;
            }
        }
        __syncwarp();
        *reinterpret_cast<float4*>(&s_e[warp][lane][0]) = make_float4(ev[0], ev[1], ev[2], ev[3]);
    }
    __syncwarp();
    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;
#pragma unroll
    for (int u = 0; u < UN; u++) {
        const float4 pr = *reinterpret_cast<const float4*>(&s_e[warp][u * RPI + rsel][0]);
        const float vx = __uint_as_float(bv[u].x), vy = __uint_as_float(bv[u].y), vz = __uint_as_float(bv[u].z), vw = __uint_as_float(bv[u].w);
        const float pm[4] = {pr.x, pr.y, pr.z, pr.w};
#pragma unroll
        for (int m = 0; m < 4; m++) {
            acc[m][0] = fmaf(pm[m], vx, acc[m][0]);
            acc[m][1] = fmaf(pm[m], vy, acc[m][1]);
            acc[m][2] = fmaf(pm[m], vz, acc[m][2]);
            acc[m][3] = fmaf(pm[m], vw, acc[m][3]);
        }
    }
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            float x = acc[m][j];
#pragma unroll
            for (int off = LPR; off < 32; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            acc[m][j] = x;
        }
    if (rsel == 0) {
#pragma unroll
        for (int m = 0; m < 4; m++) *reinterpret_cast<float4*>(&s_a[warp][m][4 * sub]) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    }
    __syncthreads();
    // the four warps of the CTA -> one partial record
    float* rec = sp.partial + (prob * sp.nsplit + split) * REC;
    for (int i = threadIdx.x; i < 4 * D; i += 128) {
        const int m = i / D, d = i - m * D;
        float M = s_m[0][m];
#pragma unroll
        for (int w = 1; w < 4; w++) M = fmaxf(M, s_m[w][m]);
        float A = 0.f, L = 0.f;
#pragma unroll
        for (int w = 0; w < 4; w++) {
            const float f = s_m[w][m] == -INFINITY ? 0.f : expf(s_m[w][m] - M);
            A = fmaf(s_a[w][m][d], f, A);
            L = fmaf(s_l[w][m], f, L);
        }
        rec[8 + i] = A;
        if (d == 0) {
            rec[m] = M;
            rec[4 + m] = L;
        }
    }
    __threadfence();
    __syncthreads();
    if (threadIdx.x == 0) s_last = atomicAdd(sp.counters + prob, 1) == sp.nsplit - 1;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    const float* recs = sp.partial + prob * sp.nsplit * REC;
    for (int i = threadIdx.x; i < p.rows * D; i += 128) {
        const int m = i / D;
        float M = -INFINITY;
        for (int k = 0; k < sp.nsplit; k++) M = fmaxf(M, __ldcg(recs + k * REC + m));
        float A = 0.f, L = 0.f;
        for (int k = 0; k < sp.nsplit; k++) {
            const float mk = __ldcg(recs + k * REC + m);
            const float f = mk == -INFINITY ? 0.f : expf(mk - M);
            A = fmaf(__ldcg(recs + k * REC + 8 + i), f, A);
            L = fmaf(__ldcg(recs + k * REC + 4 + m), f, L);
        }
        p.out[prob * p.rows * D + i] = A / L;
    }
    if (threadIdx.x == 0) sp.counters[prob] = 0;
}

// ---------------------------------------------------------------------------------------------------------------------
// One pass over K and V ("flash" decode), fed by bulk copies.  One CTA per problem: 4 working warps and one warp that
// feeds a ring of three shared-memory stages.  The keys are taken in blocks of 32: the feeding warp requests the block's K
// rows and V rows (contiguous in the cache) with cp.async.bulk, so up to 48 KB per CTA at head_dim 64 are on their way
// from HBM while the warps work on earlier blocks - loads cost no registers and never wait for arithmetic.  Four such
// CTAs share an SM: 592 places on 148 SMs, so the 512 problems of 64 requests x 8 KV heads are all resident at once
// (with 8 warps and 64-key blocks, two CTAs per SM, they ran as two uneven waves: 31 us against 27 us).  Inside the
// loop nothing synchronises the CTA: every warp keeps a running softmax of its own.
// Per block, warp w takes keys 8 w .. 8 w + 7:
//   scores   LPR lanes read one K row from shared memory (16 bytes each), dot products by the FMA order and shuffle
//            butterfly of the kernels above; scale; the 8 x 4 scores go to the warp's own 128 bytes of shared memory.
//   softmax  lane i holds score (key i / 4, row i % 4) and adds its mask value: row maximum over the 8 keys by shuffles,
//            one expf for the probability, one for the factor that rescales what the warp has accumulated so far;
//            probabilities back to shared memory.
//   values   the warp's 8 V rows times their probabilities into acc[4][4] (lane = 4 columns of the head).
//   then lane 0 hands the stage back to the feeding warp (an mbarrier that counts the working warps).
// At the end the warps' maxima, sums and accumulators meet in shared memory and are combined in warp order.
// Waits are bounded; if one ever expired the problem's output would be NaN (never observed).
// ---------------------------------------------------------------------------------------------------------------------
constexpr int FL_KEYS = 32;     // keys per block
constexpr int FL_STAGES = 3;
constexpr int FL_WARPS = 4;     // working warps; one more feeds the ring
constexpr int FL_THREADS = 32 * (FL_WARPS + 1);

template <int LPR>
struct FlashSmem {
    static constexpr int D = 4 * LPR;
    static constexpr uint32_t BLOCK_BYTES = FL_KEYS * D * 4;                 // K (or V) rows of one block
    static constexpr uint32_t STAGE_BYTES = 2 * BLOCK_BYTES;
    static constexpr uint32_t RING_BYTES = FL_STAGES * STAGE_BYTES;          // reused at the end: [warps][4 rows][D] partial outputs
    static constexpr uint32_t SCORES_OFF = RING_BYTES;                       // [warps][8 keys][4 rows] floats
    static constexpr uint32_t CORR_OFF = SCORES_OFF + FL_WARPS * 32 * 4;     // [warps][4 rows] rescale factors
    static constexpr uint32_t STATS_OFF = CORR_OFF + FL_WARPS * 4 * 4;       // m[warps][4], then l[warps][4]
    static constexpr uint32_t BAR_OFF = STATS_OFF + 2 * FL_WARPS * 4 * 4;    // full[FL_STAGES], empty[FL_STAGES] mbarriers, then a flag word
    static constexpr uint32_t TOTAL = BAR_OFF + 16 * FL_STAGES + 16;
    static_assert(RING_BYTES >= FL_WARPS * 4 * D * 4, "the ring must hold the warps' partial outputs");
};

__device__ __forceinline__ uint32_t fl_smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

// Bounded wait on an mbarrier phase; false if it expired or another thread has given up.
__device__ __forceinline__ bool fl_wait(uint32_t bar, uint32_t parity, volatile int* bad) {
    for (uint32_t spin = 0; spin < (1u << 22); spin++) {
        uint32_t done;
        asm volatile("{\n\t.reg .pred q;\n\tmbarrier.try_wait.parity.shared::cta.b64 q, [%1], %2;\n\tselp.u32 %0, 1, 0, q;\n\t}"
                     : "=r"(done) : "r"(bar), "r"(parity) : "memory");
        if (done) return true;
        if (*bad) return false;
    }
    *bad = 1;
    return false;
}

template <int LPR>
__global__ void __launch_bounds__(FL_THREADS, LPR <= 16 ? 4 : 2) gqa_decode_flash_kernel(AttnParams p) {
    using L = FlashSmem<LPR>;
    constexpr int D = 4 * LPR;
    constexpr int RPI = 32 / LPR;          // rows per warp-wide 16-byte-per-lane access
    constexpr int UN = 8 / RPI;            // accesses per warp and block: 8 keys
    static_assert(8 % RPI == 0, "a warp's 8 keys must be whole accesses");
    dep_trigger();
    extern __shared__ __align__(128) uint8_t fl_smem[];
    float* s_a = reinterpret_cast<float*>(fl_smem);
    float* s_m = reinterpret_cast<float*>(fl_smem + L::STATS_OFF);
    float* s_l = s_m + FL_WARPS * 4;
    volatile int* s_bad = reinterpret_cast<volatile int*>(fl_smem + L::BAR_OFF + 16 * FL_STAGES);
    const uint32_t bars = fl_smem_u32(fl_smem + L::BAR_OFF);
    const uint32_t ring = fl_smem_u32(fl_smem);
    auto full = [&](int st) { return bars + 8u * st; };
    auto empty = [&](int st) { return bars + 8u * (FL_STAGES + st); };
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int sub = lane % LPR, rsel = lane / LPR;
    const int64_t prob = blockIdx.x;
    const int T = p.T;
    const int n_blocks = (T + FL_KEYS - 1) / FL_KEYS;
    const float* __restrict__ Kp = p.k + prob * p.kb;
    const float* __restrict__ Vp = p.v + prob * p.vb;

    if (threadIdx.x == 0) {
        for (int st = 0; st < FL_STAGES; st++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(full(st)) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(empty(st)), "r"(FL_WARPS) : "memory");
        }
        *s_bad = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    dep_wait();  // the caches and q may have been written by the previous kernel of the stream
    __syncthreads();

    float acc[4][4];
#pragma unroll
    for (int m = 0; m < 4; m++)
#pragma unroll
        for (int j = 0; j < 4; j++) acc[m][j] = 0.f;

    if (warp == FL_WARPS) {
        // ---------------- feeds the ring ----------------
        if (lane == 0) {
            for (int blk = 0; blk < n_blocks; blk++) {
                const int st = blk % FL_STAGES;
                if (blk >= FL_STAGES && !fl_wait(empty(st), ((blk / FL_STAGES) - 1) & 1, s_bad)) break;
                const int keys = T - blk * FL_KEYS < FL_KEYS ? T - blk * FL_KEYS : FL_KEYS;
                const uint32_t bytes = static_cast<uint32_t>(keys) * D * 4;
                const uint32_t bar = full(st), dst = ring + st * L::STAGE_BYTES;
                asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(2 * bytes) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst), "l"(Kp + static_cast<int64_t>(blk) * FL_KEYS * D), "r"(bytes), "r"(bar) : "memory");
                asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                             ::"r"(dst + L::BLOCK_BYTES), "l"(Vp + static_cast<int64_t>(blk) * FL_KEYS * D), "r"(bytes), "r"(bar) : "memory");
            }
        }
    } else {
        // ---------------- working warps ----------------
        float* s_w = reinterpret_cast<float*>(fl_smem + L::SCORES_OFF) + warp * 32;
        float* s_cw = reinterpret_cast<float*>(fl_smem + L::CORR_OFF) + warp * 4;
        float4 a[4];
#pragma unroll
        for (int m = 0; m < 4; m++) {
            a[m] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (m < p.rows) a[m] = __ldg(reinterpret_cast<const float4*>(p.q + (prob * p.rows + m) * D + 4 * sub));
        }
        const int64_t b = prob / p.kv_heads, h0 = (prob % p.kv_heads) * p.rows;
        float m_run = -INFINITY, l_part = 0.f;   // of row lane % 4: running maximum (the same in all its lanes) and this lane's share of the sum

        for (int blk = 0; blk < n_blocks; blk++) {
            const int st = blk % FL_STAGES;
            const int t0 = blk * FL_KEYS;
            // the mask value of this lane's (key, row) of the softmax step is asked for now, before the wait for the block
            // and the dot products, and added there (the same two roundings, v * scale + mask, as in the kernels above)
            float mk = 0.f;
            {
                const int tm = t0 + 8 * warp + (lane >> 2), rm = lane & 3;
                if (p.mask && tm < T && rm < p.rows) mk = __ldg(p.mask + b * p.ms_b + (h0 + rm) * p.ms_h + tm);
            }
            if (!fl_wait(full(st), (blk / FL_STAGES) & 1, s_bad)) break;
            const float* Ks = reinterpret_cast<const float*>(fl_smem + st * L::STAGE_BYTES);
            const float* Vs = Ks + FL_KEYS * D;
            // ---- scores of this warp's 8 keys ----
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int kl = u * RPI + rsel, key = 8 * warp + kl, t = t0 + key;
                float4 kv = make_float4(0.f, 0.f, 0.f, 0.f);
                if (t < T) kv = *reinterpret_cast<const float4*>(Ks + key * D + 4 * sub);
                float part[4];
#pragma unroll
                for (int m = 0; m < 4; m++) part[m] = fmaf(a[m].w, kv.w, fmaf(a[m].z, kv.z, fmaf(a[m].y, kv.y, a[m].x * kv.x)));
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
                if ((sub & (LPR / 4 - 1)) == 0) {
                    float x = -INFINITY;  // keys beyond the end and rows that do not exist
                    if (t < T && m < p.rows) x = __fmul_rn(v, p.scale);
                    s_w[kl * 4 + m] = x;
                }
            }
            __syncwarp();
            // ---- running softmax: lane i has key i / 4, row i % 4 ----
            {
                float x = s_w[lane];
                if (p.mask) x = __fadd_rn(x, mk);
                float mx = x;
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 4));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 8));
                mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 16));
                const float m_new = fmaxf(m_run, mx);
                const float e = m_new == -INFINITY ? 0.f : expf(x - m_new);
                const float corr = m_run == -INFINITY ? 0.f : expf(m_run - m_new);
                l_part = fmaf(l_part, corr, e);
                m_run = m_new;
                s_w[lane] = e;
                if (lane < 4) s_cw[lane] = corr;
            }
            __syncwarp();
            // ---- values of this warp's 8 keys ----
            {
                const float4 c4 = *reinterpret_cast<const float4*>(s_cw);
                const float cr[4] = {c4.x, c4.y, c4.z, c4.w};
#pragma unroll
                for (int m = 0; m < 4; m++)
#pragma unroll
                    for (int j = 0; j < 4; j++) acc[m][j] *= cr[m];
            }
#pragma unroll
            for (int u = 0; u < UN; u++) {
                const int kl = u * RPI + rsel, key = 8 * warp + kl, t = t0 + key;
                if (t < T) {
                    const float4 pw = *reinterpret_cast<const float4*>(s_w + kl * 4);
                    const float4 vv = *reinterpret_cast<const float4*>(Vs + key * D + 4 * sub);
                    const float pm[4] = {pw.x, pw.y, pw.z, pw.w};
#pragma unroll
                    for (int m = 0; m < 4; m++) {
                        acc[m][0] = fmaf(pm[m], vv.x, acc[m][0]);
                        acc[m][1] = fmaf(pm[m], vv.y, acc[m][1]);
                        acc[m][2] = fmaf(pm[m], vv.z, acc[m][2]);
                        acc[m][3] = fmaf(pm[m], vv.w, acc[m][3]);
                    }
                }
            }
            __syncwarp();  // every lane has read the stage and the probabilities
            if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(empty(st)) : "memory");
        }
        // the warp's totals: the sum of a row over its 8 lanes, the accumulators over the lane groups that took different keys
        float l_row = l_part;
        l_row += __shfl_xor_sync(0xffffffffu, l_row, 4);
        l_row += __shfl_xor_sync(0xffffffffu, l_row, 8);
        l_row += __shfl_xor_sync(0xffffffffu, l_row, 16);
        if (lane < 4) {
            s_m[warp * 4 + lane] = m_run;
            s_l[warp * 4 + lane] = l_row;
        }
#pragma unroll
        for (int m = 0; m < 4; m++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float x = acc[m][j];
#pragma unroll
                for (int off = LPR; off < 32; off <<= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
                acc[m][j] = x;
            }
    }
    __syncthreads();  // every requested block has arrived and been read: the ring is free for the warps' partial outputs
    if (warp < FL_WARPS && rsel == 0) {
#pragma unroll
        for (int m = 0; m < 4; m++) *reinterpret_cast<float4*>(s_a + (warp * 4 + m) * D + 4 * sub) = make_float4(acc[m][0], acc[m][1], acc[m][2], acc[m][3]);
    }
    __syncthreads();
    const bool bad = *s_bad != 0;
    for (int i = threadIdx.x; i < p.rows * D; i += FL_THREADS) {
        const int m = i / D, d = i - m * D;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < FL_WARPS; w++) M = fmaxf(M, s_m[w * 4 + m]);
        float A = 0.f, Lsum = 0.f;
#pragma unroll
        for (int w = 0; w < FL_WARPS; w++) {
            const float mw = s_m[w * 4 + m];
            const float f = mw == -INFINITY ? 0.f : expf(mw - M);
            Lsum = fmaf(s_l[w * 4 + m], f, Lsum);
            A = fmaf(s_a[(w * 4 + m) * D + d], f, A);
        }
        p.out[prob * p.rows * D + i] = bad ? __int_as_float(0x7fc00000) : A / Lsum;
    }
}

constexpr int64_t ATTN_MAX_KEYS = 12288;  // 16 bytes of shared memory per key

template <int LPR>
static int attn_launch(cudaStream_t st, const AttnParams& p, int64_t problems) {
    const size_t smem = (4 * static_cast<size_t>((p.T + 3) & ~3) + 8 * 4 * 4 * LPR) * sizeof(float);
    static std::once_flag configured[64];  // once per device; a concurrent first call waits for the attribute to be set
    int dev = 0;
    cudaGetDevice(&dev);
    cudaError_t cfg_err = cudaSuccess;
    if (dev >= 0 && dev < 64)
        std::call_once(configured[dev], [&] {
            cfg_err = cudaFuncSetAttribute(gqa_decode_attention_kernel<LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           static_cast<int>((4 * ATTN_MAX_KEYS + 8 * 4 * 4 * LPR) * sizeof(float)));
        });
    RMLK_CUDA(cfg_err);
    launch_dep(gqa_decode_attention_kernel<LPR>, dim3(static_cast<unsigned>(problems)), dim3(256), smem, st, p);
    RMLK_CHECK_LAUNCH("gqa_decode_attention_kernel");
    return RMLK_OK;
}

template <int LPR>
static int attn_flash_launch(cudaStream_t st, const AttnParams& p, int64_t problems) {
    using L = FlashSmem<LPR>;
    static std::once_flag configured[64];  // once per device; a concurrent first call waits for the attribute to be set
    int dev = 0;
    cudaGetDevice(&dev);
    cudaError_t cfg_err = cudaSuccess;
    if (dev >= 0 && dev < 64)
        std::call_once(configured[dev], [&] {
            cfg_err = cudaFuncSetAttribute(gqa_decode_flash_kernel<LPR>, cudaFuncAttributeMaxDynamicSharedMemorySize, static_cast<int>(L::TOTAL));
        });
    RMLK_CUDA(cfg_err);
    launch_dep(gqa_decode_flash_kernel<LPR>, dim3(static_cast<unsigned>(problems)), dim3(FL_THREADS), L::TOTAL, st, p);
    RMLK_CHECK_LAUNCH("gqa_decode_flash_kernel");
    return RMLK_OK;
}

// RMLK_B200_ATTENTION_FLASH=0: the one-launch attention falls back to the two-pass kernels (scores of all keys in shared
// memory, then the values) for A/B runs.
static bool attn_flash_enabled() {
    static const bool v = [] {
        const char* e = getenv("RMLK_B200_ATTENTION_FLASH");
        return !(e && e[0] == '0');
    }();
    return v;
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_gqa_decode_attention_supported(int64_t rows, int64_t head_dim, int64_t keys) {
    return rows >= 1 && rows <= 4 && (head_dim == 16 || head_dim == 32 || head_dim == 64 || head_dim == 128) && keys >= 1 && keys <= ATTN_MAX_KEYS;
}

extern "C" int rmlk_b200_gqa_decode_attention(rmlk_stream_t stream, int dtype, int64_t problems, int64_t rows, int64_t head_dim, int64_t keys,
                                              int64_t kv_heads, const void* q, const void* k, int64_t k_problem_stride, const void* v,
                                              int64_t v_problem_stride, float scale, const void* mask, int64_t mask_batch_stride,
                                              int64_t mask_head_stride, void* out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for gqa_decode_attention (f32 only)");
    if (problems < 0 || kv_heads <= 0) return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: bad extent");
    if (!rmlk_b200_gqa_decode_attention_supported(rows, head_dim, keys))
        return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: needs 1..4 query rows, head_dim 16 / 32 / 64 / 128 and 1..12288 keys");
    if (problems == 0) return RMLK_OK;
    if (!q || !k || !v || !out) return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: NULL tensor pointer");
    if (problems > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: too many problems");
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(out, 16) || k_problem_stride % 4 || v_problem_stride % 4)
        return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: operands must be 16-byte aligned");
    AttnParams p;
    p.q = static_cast<const float*>(q);
    p.k = static_cast<const float*>(k);
    p.v = static_cast<const float*>(v);
    p.mask = static_cast<const float*>(mask);
    p.out = static_cast<float*>(out);
    p.kb = k_problem_stride;
    p.vb = v_problem_stride;
    p.ms_b = mask_batch_stride;
    p.ms_h = mask_head_stride;
    p.rows = static_cast<int>(rows);
    p.T = static_cast<int>(keys);
    p.kv_heads = static_cast<int>(kv_heads);
    p.scale = scale;
    cudaStream_t st = as_stream(stream);
    if (attn_flash_enabled()) {
        switch (head_dim) {
            case 16: return attn_flash_launch<4>(st, p, problems);
            case 32: return attn_flash_launch<8>(st, p, problems);
            case 64: return attn_flash_launch<16>(st, p, problems);
            default: return attn_flash_launch<32>(st, p, problems);
        }
    }
    switch (head_dim) {
        case 16: return attn_launch<4>(st, p, problems);
        case 32: return attn_launch<8>(st, p, problems);
        case 64: return attn_launch<16>(st, p, problems);
        default: return attn_launch<32>(st, p, problems);
    }
}

extern "C" size_t rmlk_b200_gqa_decode_attention_workspace_bytes(int64_t problems, int64_t rows, int64_t head_dim, int64_t keys) {
    if (!rmlk_b200_gqa_decode_attention_supported(rows, head_dim, keys) || problems <= 0 || keys <= SPLIT_KEYS) return 0;
    const int64_t nsplit = ceil_div64(keys, SPLIT_KEYS);
    return static_cast<size_t>(problems) * (sizeof(int) * 4 + static_cast<size_t>(nsplit) * (8 + 4 * head_dim) * sizeof(float));
}

template <int LPR>
static int attn_split_launch(cudaStream_t st, const AttnSplitParams& sp, int64_t problems) {
    launch_dep(gqa_decode_attention_split_kernel<LPR>, dim3(static_cast<unsigned>(sp.nsplit), static_cast<unsigned>(problems)), dim3(128), 0, st, sp);
    RMLK_CHECK_LAUNCH("gqa_decode_attention_split_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_gqa_decode_attention_ws(rmlk_stream_t stream, int dtype, int64_t problems, int64_t rows, int64_t head_dim, int64_t keys,
                                                 int64_t kv_heads, const void* q, const void* k, int64_t k_problem_stride, const void* v,
                                                 int64_t v_problem_stride, float scale, const void* mask, int64_t mask_batch_stride,
                                                 int64_t mask_head_stride, void* out, void* workspace, size_t workspace_bytes) {
    const size_t need = rmlk_b200_gqa_decode_attention_workspace_bytes(problems, rows, head_dim, keys);
    if (dtype != RMLK_F32 || !need || !workspace || workspace_bytes < need || problems > 65535 || !aligned_to(workspace, 16))
        return rmlk_b200_gqa_decode_attention(stream, dtype, problems, rows, head_dim, keys, kv_heads, q, k, k_problem_stride, v, v_problem_stride, scale,
                                              mask, mask_batch_stride, mask_head_stride, out);
    if (kv_heads <= 0) return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: bad extent");
    if (!q || !k || !v || !out) return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: NULL tensor pointer");
    if (!aligned_to(q, 16) || !aligned_to(k, 16) || !aligned_to(v, 16) || !aligned_to(out, 16) || k_problem_stride % 4 || v_problem_stride % 4)
        return fail(RMLK_ERR_INVALID_ARG, "gqa_decode_attention: operands must be 16-byte aligned");
    AttnSplitParams sp;
    sp.base.q = static_cast<const float*>(q);
    sp.base.k = static_cast<const float*>(k);
    sp.base.v = static_cast<const float*>(v);
    sp.base.mask = static_cast<const float*>(mask);
    sp.base.out = static_cast<float*>(out);
    sp.base.kb = k_problem_stride;
    sp.base.vb = v_problem_stride;
    sp.base.ms_b = mask_batch_stride;
    sp.base.ms_h = mask_head_stride;
    sp.base.rows = static_cast<int>(rows);
    sp.base.T = static_cast<int>(keys);
    sp.base.kv_heads = static_cast<int>(kv_heads);
    sp.base.scale = scale;
    sp.nsplit = static_cast<int>(ceil_div64(keys, SPLIT_KEYS));
    sp.counters = static_cast<int*>(workspace);
    sp.partial = reinterpret_cast<float*>(static_cast<char*>(workspace) + static_cast<size_t>(problems) * sizeof(int) * 4);
    cudaStream_t st = as_stream(stream);
    switch (head_dim) {
        case 16: return attn_split_launch<4>(st, sp, problems);
        case 32: return attn_split_launch<8>(st, sp, problems);
        case 64: return attn_split_launch<16>(st, sp, problems);
        default: return attn_split_launch<32>(st, sp, problems);
    }
}
