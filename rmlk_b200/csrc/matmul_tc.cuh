// Device side of the tensor-core MatMul (see matmul_tc.cu for the overview).
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace rmlk {
namespace tc {

constexpr int BK = 32;    // fp32 elements per k-block: one 128-byte row
constexpr int BN = 128;   // weight columns per CTA = MMA M = TMEM lanes
// weight-TMA warp, MMA warp, G x 4 converter / epilogue warps, activation-TMA warp
constexpr int threads_for(int groups) { return 64 + 128 * groups + 32; }
constexpr uint32_t SPIN_LIMIT = 1u << 20;
constexpr uint32_t TF32_MASK = 0xffffe000u;  // sign, exponent and the 10 mantissa bits a tf32 MMA operand keeps

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
// Bounded wait.  Returns false if the wait expired or another thread of the CTA already gave up.
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

// D[tmem] (+)= A[tmem] x B[smem descriptor], kind::tf32, issued by one thread.
__device__ __forceinline__ void tc_mma_tf32_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], %2, %3, {%5, %6, %7, %8}, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}

// The same MMA with the shared-memory descriptor handed over as two 32-bit halves and the accumulator always added to:
// the issuing thread keeps the constant upper half in a register and only adds to the lower one.
__device__ __forceinline__ void tc_mma_tf32_ts_acc(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_desc_lo, uint32_t b_desc_hi, uint32_t idesc) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t.reg .b64 d;\n\t"
        "mov.b64 d, {%2, %3};\n\t"
        "setp.eq.b32 p, 0, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], [%1], d, %4, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "r"(b_desc_lo), "r"(b_desc_hi), "r"(idesc)
        : "memory");
}

// K-major shared-memory operand descriptor, 128-byte swizzle, descriptor version 1.
__device__ __forceinline__ uint64_t smem_desc_k128(uint32_t addr) {
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr >> 4) & 0x3fff);
    d |= static_cast<uint64_t>(1) << 16;            // leading byte offset (unused for swizzled K-major): 16 B
    d |= static_cast<uint64_t>(1024 >> 4) << 32;    // stride between 8-row groups: 1024 B
    d |= 1ull << 46;                                 // version
    d |= 2ull << 61;                                 // SWIZZLE_128B
    return d;
}

__device__ __forceinline__ uint32_t to_tf32(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}

__device__ __forceinline__ void tmem_ld_x32(uint32_t taddr, uint32_t (&r)[32]) {
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

__device__ __forceinline__ void tmem_st_x16(uint32_t taddr, const uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
        "{%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
        ::"r"(taddr), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3]), "r"(r[4]), "r"(r[5]), "r"(r[6]), "r"(r[7]), "r"(r[8]), "r"(r[9]),
          "r"(r[10]), "r"(r[11]), "r"(r[12]), "r"(r[13]), "r"(r[14]), "r"(r[15])
        : "memory");
}

// ---- thread-block cluster helpers (split-K partial sums exchanged through distributed shared memory) ----
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// Executed by every thread of every CTA of the cluster.
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\n\tbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// Address of this CTA's shared-memory location `addr` in the CTA of rank `cta` of the same cluster.
__device__ __forceinline__ uint32_t mapa_shared(uint32_t addr, uint32_t cta) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(addr), "r"(cta));
    return r;
}
__device__ __forceinline__ void st_shared_cluster_f32(uint32_t addr, float v) {
    asm volatile("st.shared::cluster.f32 [%0], %1;" ::"r"(addr), "f"(v) : "memory");
}

constexpr int MAX_PEERS = 7;  // other ranks of one NVLink domain (8 GPUs)

struct TcParams {
    int cluster_reduce;     // ksplit CTAs form a cluster along grid y and add their partial sums on chip
    float* out;             // C, or the split-K scratch [ksplit][M][N]
    int64_t M, N, K;
    int64_t ldc;            // elements between rows of `out` (N, unless C is a block of columns of a wider matrix)
    int k_iters_per_split;  // k-blocks per split
    int k_iters_total;
    int ksplit;
    int* status;
    int w_static;           // the weights are not written by work still in flight: their loads need not wait for the previous kernel
    // Column-split MatMul across GPUs: every finished element of C is also stored at the same offset from each of these
    // bases - the other ranks' output buffers, mapped into this GPU's address space (ordinary stores that cross NVLink).
    int n_peer;
    float* peer_out[MAX_PEERS];
};

// Shared memory: a ring of SW raw weight blocks (freed as soon as the converters have moved a block into TMEM) and a
// ring of SA activation blocks (raw tile + its lo twin, read by the MMA from shared memory, freed when the MMAs of
// that k-block complete).  TMEM: two accumulator blocks + one (hi, lo) weight block per activation stage.
template <int MT, int SW, int SA>
struct SmemLayout {
    static constexpr uint32_t W_BYTES = BK * BN * 4;   // 16 KB raw weights: [32 k][128 n] row-major, unswizzled
    static constexpr uint32_t A_BYTES = MT * BK * 4;   // activations [MT rows][32 k], 128-byte swizzled
    static constexpr uint32_t A_STAGE_BYTES = 2 * A_BYTES;
    static constexpr uint32_t A_OFFSET = SW * W_BYTES;
    static constexpr uint32_t TILE_BYTES = SW * W_BYTES + SA * A_STAGE_BYTES;
    static constexpr uint32_t BAR_OFFSET = TILE_BYTES;
    static constexpr uint32_t N_BARS = 2 * SW + 3 * SA + 1;
    static constexpr uint32_t TOTAL = TILE_BYTES + 8 * N_BARS + 32 + 1024;  // barriers, TMEM slot + abort flag, slack for 1024-byte alignment
    static constexpr uint32_t TMEM_COLS_USED = 2 * MT + 64 * SA;
    static constexpr uint32_t TMEM_COLS = TMEM_COLS_USED <= 64 ? 64 : TMEM_COLS_USED <= 128 ? 128 : TMEM_COLS_USED <= 256 ? 256 : 512;
    static_assert(TMEM_COLS_USED <= 512, "TMEM budget exceeded");
    static_assert(TOTAL <= 227 * 1024, "shared memory budget exceeded");
};

}  // namespace tc
}  // namespace rmlk
