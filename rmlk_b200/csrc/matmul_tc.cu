// fp32 MatMul on the 5th-generation tensor cores: tcgen05.mma kind::tf32 with a 3xTF32 split, operands
// staged by TMA, accumulators in TMEM.  C[M,N] = A[M,K] x W[K,N], all row-major fp32.
//
// Orientation.  The weight matrix W is the large, streamed operand and its N dimension is contiguous,
// so it is fed as the MMA's *A* operand in MN-major form: one CTA owns 128 columns of W (MMA M = 128,
// one TMEM lane per column) and a tile of MT <= 128 rows of the activation matrix, which is the MMA's
// K-major *B* operand (MMA N = MT).  The accumulator D[n][m] therefore sits in TMEM as 128 lanes x MT
// fp32 columns, i.e. transposed with respect to C; the epilogue writes C[m][n0 + lane], which is
// coalesced across the lanes of a warp.
//
// 3xTF32.  An fp32 value x is split into hi = x with the low 13 mantissa bits cleared (exactly a tf32)
// and lo = x - hi (exact in fp32; it is rounded to tf32 by the tensor core).  Per k-block three MMAs
// accumulate hi*hi + hi*lo + lo*hi in fp32; the dropped lo*lo term is below 2^-20 relative.
//
// Pipeline (STAGES deep, one output tile per CTA, K optionally split across CTAs):
//   warp 0      TMA producer: per k-block of 32, four 32x32 boxes of W and one 32xMT box of A, 128-byte
//               swizzled, completing on full[s]
//   warps 2-5   converters: read the raw fp32 tiles, write hi back in place and lo into the twin buffer at
//               the same (swizzled) offsets, then fence the generic->async proxy and arrive on conv[s]
//   warp 1      MMA issuer (one thread): 4 k-steps x 3 tcgen05.mma per stage, tcgen05.commit -> empty[s];
//               after the last stage tcgen05.commit -> accum
//   warps 2-5   epilogue: tcgen05.ld 32 lanes x 32 columns at a time, store to C (or to the split-K scratch)
//
// Every mbarrier wait is bounded: on expiry the thread raises a block-wide abort flag, records
// RMLK_ERR_TIMEOUT in the caller's status word, and all roles fall through to the common exit where
// TMEM is released.  Every TMA load targets this CTA's own shared memory; the kernel runs as single-CTA clusters.
#include <cuda.h>

#include "common.cuh"

namespace rmlk {
namespace tc {

constexpr int BK = 32;    // fp32 elements per k-block: one 128-byte swizzle row
constexpr int BN = 128;   // weight columns per CTA = MMA M
constexpr int THREADS = 192;
constexpr uint32_t SPIN_LIMIT = 1u << 20;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return static_cast<uint32_t>(__cvta_generic_to_shared(p)); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint32_t bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait.  Returns false if the wait expired or another thread already aborted.
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag, int* status) {
    for (uint32_t i = 0; i < SPIN_LIMIT; i++) {
        if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
    }
    *abort_flag = 1;
    if (status) atomicExch(status, RMLK_ERR_TIMEOUT);
    return false;
}

__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(reinterpret_cast<uint64_t>(map)), "r"(x), "r"(y), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void fence_proxy_async() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tc_commit(uint32_t bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

__device__ __forceinline__ void tc_mma_tf32(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// Shared-memory matrix descriptor, 128-byte swizzle, descriptor version 1 (Blackwell).
// layout: 2 = 128-byte swizzle in 16-byte units (K-major operands), 1 = 128-byte swizzle in 32-byte units, the
// form 32-bit MN-major operands need (TMA: CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B).
__device__ __forceinline__ uint64_t smem_desc(uint32_t addr, uint32_t lbo_bytes, uint32_t sbo_bytes, uint64_t layout = 2) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= static_cast<uint64_t>((sbo_bytes >> 4) & 0x3fff) << 32;
    d |= 1ull << 46;   // version
    d |= layout << 61;
    return d;
}

__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]), "=r"(r[9]),
          "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]),
          "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]),
          "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}

struct TcParams {
    float* out;            // C, or the split-K scratch [ksplit][M][N]
    int64_t M, N, K;
    int k_iters_per_split; // k-blocks per split
    int k_iters_total;
    int ksplit;
    int* status;
    int debug;
};

template <int MT, int STAGES>
struct SmemLayout {
    static constexpr uint32_t W_BYTES = BK * BN * 4;      // 16 KB: 4 slabs of [32 k][32 n]
    static constexpr uint32_t A_BYTES = MT * BK * 4;      // [MT rows][32 k]
    static constexpr uint32_t STAGE_BYTES = 2 * W_BYTES + 2 * A_BYTES;
    static constexpr uint32_t TILE_BYTES = STAGES * STAGE_BYTES;
    static constexpr uint32_t BAR_OFFSET = TILE_BYTES;
    static constexpr uint32_t TOTAL = TILE_BYTES + 256 + 1024;  // barriers + slack for 1024-byte alignment
};

template <int MT, int STAGES>
__global__ void __launch_bounds__(THREADS, 1) tc_gemm_kernel(const __grid_constant__ CUtensorMap tmW,
                                                              const __grid_constant__ CUtensorMap tmA, TcParams p) {
    using L = SmemLayout<MT, STAGES>;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFFSET;
    // barrier slots (8 bytes each): full[s], conv[s], empty[s], accum; then tmem slot and abort flag
    auto full_bar = [&](int s) { return bars + 8u * s; };
    auto conv_bar = [&](int s) { return bars + 8u * (STAGES + s); };
    auto empty_bar = [&](int s) { return bars + 8u * (2 * STAGES + s); };
    const uint32_t accum_bar = bars + 8u * (3 * STAGES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::BAR_OFFSET + 8 * (3 * STAGES + 1));
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFFSET + 8 * (3 * STAGES + 1) + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * BN;
    const int split = blockIdx.y;
    const int m0 = blockIdx.z * MT;
    const int it_begin = split * p.k_iters_per_split;
    int n_iters = p.k_iters_total - it_begin;
    if (n_iters > p.k_iters_per_split) n_iters = p.k_iters_per_split;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; s++) {
            mbar_init(full_bar(s), 1);
            mbar_init(conv_bar(s), 128);
            mbar_init(empty_bar(s), 1);
        }
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(MT) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ---------------- TMA producer ----------------
        if (lane == 0) {
            for (int it = 0; it < n_iters; it++) {
                const int s = it % STAGES;
                if (it >= STAGES && !mbar_wait(empty_bar(s), ((it / STAGES) - 1) & 1, abort_flag, p.status)) break;
                const uint32_t st = base + s * L::STAGE_BYTES;
                const int k0 = (it_begin + it) * BK;
                mbar_expect_tx(full_bar(s), L::W_BYTES + L::A_BYTES);
#pragma unroll
                for (int j = 0; j < 4; j++) tma_load_2d(st + j * 4096, &tmW, n0 + 32 * j, k0, full_bar(s));
                tma_load_2d(st + 2 * L::W_BYTES, &tmA, k0, m0, full_bar(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // instruction descriptor: D fp32, A/B tf32, A (weights) MN-major, B (activations) K-major, M = 128, N = MT
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | (1u << 15) | (0u << 16) | ((MT >> 3) << 17) | ((BN >> 4) << 24);
            bool ok = true;
            for (int it = 0; it < n_iters && ok; it++) {
                const int s = it % STAGES;
                ok = mbar_wait(conv_bar(s), (it / STAGES) & 1, abort_flag, p.status);
                if (!ok) break;
                tc_fence_after();
                const uint32_t st = base + s * L::STAGE_BYTES;
                const uint32_t w_hi = st, w_lo = st + L::W_BYTES, a_hi = st + 2 * L::W_BYTES, a_lo = a_hi + L::A_BYTES;
#pragma unroll
                for (int kk = 0; kk < BK / 8; kk++) {
                    // weights (MN-major, 32-byte swizzle atoms): slabs of 32 columns 4096 B apart (LBO), groups of
                    // 4 k-rows 512 B apart (SBO); a k-step of 8 rows advances the start by 1024 B
                    const uint64_t dw_hi = smem_desc(w_hi + kk * 1024, 4096, 512, 1);
                    const uint64_t dw_lo = smem_desc(w_lo + kk * 1024, 4096, 512, 1);
                    // activations: 8-row groups 1024 B apart (SBO), a k-step is 32 B inside the swizzled row
                    const uint64_t da_hi = smem_desc(a_hi + kk * 32, 16, 1024);
                    const uint64_t da_lo = smem_desc(a_lo + kk * 32, 16, 1024);
                    if (p.debug == 6) {
                        constexpr uint32_t idk = (1u << 4) | (2u << 7) | (2u << 10) | ((MT >> 3) << 17) | ((BN >> 4) << 24);
                        tc_mma_tf32(tmem_base, da_hi, da_hi, idk, (it > 0 || kk > 0) ? 1u : 0u);
                        continue;
                    }
                    if (p.debug == 7) continue;
                    tc_mma_tf32(tmem_base, dw_lo, da_hi, idesc, (it > 0 || kk > 0) ? 1u : 0u);
                    tc_mma_tf32(tmem_base, dw_hi, da_lo, idesc, 1u);
                    tc_mma_tf32(tmem_base, dw_hi, da_hi, idesc, 1u);
                }
                tc_commit(empty_bar(s));
            }
            tc_commit(accum_bar);
        }
    } else {
        // ---------------- converters, then epilogue ----------------
        const int t = threadIdx.x - 64;  // 0..127
        constexpr int W_CHUNKS = L::W_BYTES / 16, A_CHUNKS = L::A_BYTES / 16;
        bool ok = true;
        for (int it = 0; it < n_iters && ok; it++) {
            const int s = it % STAGES;
            ok = mbar_wait(full_bar(s), (it / STAGES) & 1, abort_flag, p.status);
            if (!ok) break;
            uint8_t* st = base_ptr + s * L::STAGE_BYTES;
            auto split_chunks = [&](uint8_t* hi, uint8_t* lo, int chunks) {
#pragma unroll 4
                for (int c = t; c < chunks; c += 128) {
                    uint4 v = *reinterpret_cast<uint4*>(hi + 16 * c);
                    uint4 h, l;
                    h.x = v.x & 0xffffe000u; h.y = v.y & 0xffffe000u; h.z = v.z & 0xffffe000u; h.w = v.w & 0xffffe000u;
                    l.x = __float_as_uint(__uint_as_float(v.x) - __uint_as_float(h.x));
                    l.y = __float_as_uint(__uint_as_float(v.y) - __uint_as_float(h.y));
                    l.z = __float_as_uint(__uint_as_float(v.z) - __uint_as_float(h.z));
                    l.w = __float_as_uint(__uint_as_float(v.w) - __uint_as_float(h.w));
                    *reinterpret_cast<uint4*>(hi + 16 * c) = h;
                    *reinterpret_cast<uint4*>(lo + 16 * c) = l;
                }
            };
            split_chunks(st, st + L::W_BYTES, W_CHUNKS);
            split_chunks(st + 2 * L::W_BYTES, st + 2 * L::W_BYTES + L::A_BYTES, A_CHUNKS);
            fence_proxy_async();
            mbar_arrive(conv_bar(s));
        }
        if (ok) ok = mbar_wait(accum_bar, 0, abort_flag, p.status);
        if (ok) {
            tc_fence_after();
            const int sub = warp & 3;                 // TMEM sub-partition this warp may read
            const int64_t n = n0 + sub * 32 + lane;   // weight column held by this thread's TMEM lane
            float* out = p.out + (p.ksplit > 1 ? static_cast<int64_t>(split) * p.M * p.N : 0);
#pragma unroll
            for (int c0 = 0; c0 < MT; c0 += 32) {
                uint32_t r[32];
                if (p.debug == 5) {
                    const uint32_t val = __float_as_uint(1000.0f * sub + lane + 0.01f * c0);
                    asm volatile("tcgen05.st.sync.aligned.32x32b.x1.b32 [%0], {%1};" ::"r"(tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + c0 + 3), "r"(val) : "memory");
                    asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                }
                tmem_ld_32x32(tmem_base + (static_cast<uint32_t>(sub * 32) << 16) + c0, r);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int64_t m = m0 + c0 + j;
                    float v = __uint_as_float(r[j]);
                    if (p.debug == 1) v = 7.0f;
                    if (p.debug == 2) v = static_cast<float>(tmem_base);
                    if (p.debug == 3) v = reinterpret_cast<float*>(base_ptr)[((c0 + j) * 128 + sub * 32 + lane) % 4096];
                    if (p.debug == 4) v = reinterpret_cast<float*>(base_ptr + 2 * L::W_BYTES)[((c0 + j) * 32 + lane) % (MT * 32)];
                    if (m < p.M) out[m * p.N + n] = v;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(MT) : "memory");
    }
}

// ---- host side ---------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    }
    return fn;
}

static bool make_map_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swizzle) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {inner * 4};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MT, int STAGES>
static int launch(cudaStream_t st, const CUtensorMap& tmW, const CUtensorMap& tmA, const TcParams& p, dim3 grid) {
    using L = SmemLayout<MT, STAGES>;
    static bool configured[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !configured[dev]) {
        RMLK_CUDA(cudaFuncSetAttribute(tc_gemm_kernel<MT, STAGES>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL));
        configured[dev] = true;
    }
    tc_gemm_kernel<MT, STAGES><<<grid, THREADS, L::TOTAL, st>>>(tmW, tmA, p);
    RMLK_CHECK_LAUNCH("tc_gemm_kernel");
    return RMLK_OK;
}

}  // namespace tc

bool tc_enabled() {
    static int v = -1;
    if (v < 0) {
        const char* e = getenv("RMLK_B200_NO_TC");
        v = (e && e[0] == '1') ? 0 : 1;
    }
    return v == 1;
}

// Eligibility of the tensor-core path for C[M,N] = A[M,K] x W[K,N].
bool tc_matmul_eligible(int64_t m, int64_t n, int64_t k, const void* a, const void* w, const void* c) {
    return tc_enabled() && m > 16 && (n % tc::BN == 0) && (k % tc::BK == 0) && k >= tc::BK && aligned_to(a, 16) && aligned_to(w, 16) &&
           aligned_to(c, 16) && n < (1ll << 31) && k < (1ll << 31) && m < (1ll << 31) && tc::encode_fn() != nullptr;
}

int tc_matmul_plan(int64_t m, int64_t n, int64_t k) {
    const int mt = m <= 64 ? 64 : 128;
    const int64_t tiles = (n / tc::BN) * ceil_div64(m, mt);
    const int64_t k_iters = k / tc::BK;
    int64_t s = sm_count() / tiles;  // fill the GPU with one wave of CTAs, never spill into a second
    const int64_t max_s = k_iters / 8 > 0 ? k_iters / 8 : 1;  // at least 8 k-blocks per split
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    return static_cast<int>(s > 32 ? 32 : s);
}

size_t tc_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    const int s = tc_matmul_plan(m, n, k);
    return s > 1 ? static_cast<size_t>(s) * m * n * sizeof(float) : 0;
}

// Launches the tensor-core GEMM.  `ksplit_out` tells the caller how many partial slabs were written to
// `workspace` (1 = result is already in c).
int tc_matmul(cudaStream_t st, int64_t m, int64_t n, int64_t k, const float* a, const float* w, float* c, void* workspace,
              size_t workspace_bytes, int* status, int* ksplit_out) {
    const int mt = m <= 64 ? 64 : 128;
    int ksplit = tc_matmul_plan(m, n, k);
    if (ksplit > 1 && (!workspace || workspace_bytes < static_cast<size_t>(ksplit) * m * n * sizeof(float))) ksplit = 1;
    const int k_iters = static_cast<int>(k / tc::BK);
    const int per = static_cast<int>(ceil_div64(k_iters, ksplit));
    ksplit = static_cast<int>(ceil_div64(k_iters, per));
    CUtensorMap tmW, tmA;
    if (!tc::make_map_2d(&tmW, w, static_cast<uint64_t>(n), static_cast<uint64_t>(k), 32, 32, CU_TENSOR_MAP_SWIZZLE_128B_ATOM_32B) ||
        !tc::make_map_2d(&tmA, a, static_cast<uint64_t>(k), static_cast<uint64_t>(m), 32, static_cast<uint32_t>(mt), CU_TENSOR_MAP_SWIZZLE_128B))
        return fail(RMLK_ERR_INTERNAL, "matmul: cuTensorMapEncodeTiled failed");
    tc::TcParams p;
    p.out = ksplit > 1 ? static_cast<float*>(workspace) : c;
    p.M = m; p.N = n; p.K = k;
    p.k_iters_per_split = per;
    p.k_iters_total = k_iters;
    p.ksplit = ksplit;
    p.status = status;
    { const char* e = getenv("RMLK_B200_TC_DEBUG"); p.debug = e ? atoi(e) : 0; }
    dim3 grid(static_cast<unsigned>(n / tc::BN), static_cast<unsigned>(ksplit), static_cast<unsigned>(ceil_div64(m, mt)));
    *ksplit_out = ksplit;
    if (mt == 64) return tc::launch<64, 4>(st, tmW, tmA, p, grid);
    return tc::launch<128, 3>(st, tmW, tmA, p, grid);
}

}  // namespace rmlk
