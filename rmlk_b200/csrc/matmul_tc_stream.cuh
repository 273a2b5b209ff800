// tc_stream_kernel: the tensor-core MatMul as a persistent kernel - one CTA per SM, each working through a contiguous
// range of (tile, k-block) units.  Same operand path per k-block as tc_gemm_kernel (matmul_tc_kernel.cuh): W by TMA
// into a shared-memory ring, moved by converter warps into TMEM as tf32 hi / lo, activations by TMA into a second
// ring with a lo twin, tcgen05.mma kind::tf32 with the weights read from TMEM.  What is new:
//
//  * The work is the sequence of all k-blocks of all [MT x 128] tiles of C, tile after tile; CTA c of G takes units
//    [units * c / G, units * (c + 1) / G).  A range may start and end inside a tile ("stream-K"), so every SM streams
//    the same number of weight bytes whatever the tile count (128 tiles on 148 SMs, 16 tiles of a long K, 6.77 waves of
//    the lm_head), and the rings never drain between tiles: producers, converters and the MMA thread just keep going.
//  * Four dedicated epilogue warps: when a segment (the part of a tile a CTA computed) is complete they pull its
//    accumulators into registers and hand the TMEM block straight back, so the MMAs of the next segment run while the
//    results are being stored.
//  * A segment that covers the whole K of its tile is stored to C directly.  Otherwise the CTAs that share the tile (a
//    group of P consecutive CTAs) each store their partial tile to a slot of the scratch buffer and raise a flag for
//    every member; at the very end of its life each member waits for the group's flags and adds up its share of the
//    tile's rows (row m belongs to member m % P) over the P slots in CTA order - a fixed order, so the result is
//    deterministic - and writes those rows of C.  A CTA publishes all its partial tiles before it waits for anybody,
//    so no CTA can wait for one that waits for it.  Every wait is bounded.
//  * Flags carry a per-launch token and are cleared by their reader, so the scratch needs no initialisation and a
//    captured launch can be replayed.
//  * hi x [hi; lo] is issued as one MMA with N = 2 MT (an instruction costs about 140-170 cycles whatever its N, so
//    the instruction count per k-block - two per k-step - is what bounds this kernel at small M); the third product,
//    lo x hi, is added into the hi x lo block: the tensor core truncates when it adds into its fp32 accumulator, and
//    keeping the small products out of the large hi x hi sums halves that error.
#pragma once

#include "matmul_tc.cuh"

namespace rmlk {
namespace tc {

constexpr int STREAM_THREADS = 512;   // 16 warps: W TMA, MMA, A TMA, (idle), 8 converter warps, 4 epilogue warps
constexpr int STREAM_MAX_GROUP = 16;  // CTAs that may share one tile

struct StreamParams {
    float* out;
    int64_t M, N, K, ldc;
    int k_iters;    // k-blocks per tile (K / 32)
    int m_tiles;    // row tiles per column block
    int64_t units;  // work units: tiles * k_iters / gran
    int gran;       // k-blocks per unit: 1 (a range may cut a tile) or k_iters (whole tiles only)
    int strided;    // whole tiles dealt out round-robin: CTA c takes tiles c, c + G, c + 2 G, ... (the CTAs then read adjacent
                    // 512-byte pieces of the same rows of W at the same time, which is what DRAM likes); units = tiles
    float* slots;   // [2 * gridDim.x][MT * 128] partial tiles
    unsigned long long* flags;  // [2 * gridDim.x][STREAM_MAX_GROUP]
    unsigned long long token;
    int* status;
    int w_static;
    int mma_mode;
    int n_peer;                    // column-split MatMul across GPUs: finished rows of C also go to the other ranks' buffers
    float* peer_out[MAX_PEERS];
};

template <int MT, int SW, int SA>
struct StreamSmem {
    static constexpr uint32_t W_BYTES = BK * BN * 4;
    static constexpr uint32_t A_BYTES = MT * BK * 4;
    static constexpr uint32_t A_STAGE_BYTES = 2 * A_BYTES;
    static constexpr uint32_t A_OFFSET = SW * W_BYTES;
    static constexpr uint32_t TILE_BYTES = SW * W_BYTES + SA * A_STAGE_BYTES;
    static constexpr uint32_t BAR_OFFSET = TILE_BYTES;
    static constexpr uint32_t N_BARS = 2 * SW + 3 * SA + 2;  // w_full, w_empty, a_full, conv, mma_done, acc_full, acc_empty
    static constexpr uint32_t TOTAL = TILE_BYTES + 8 * N_BARS + 32 + 1024;
    static constexpr uint32_t TMEM_COLS_USED = 2 * MT + 64 * SA;
    static constexpr uint32_t TMEM_COLS = TMEM_COLS_USED <= 64 ? 64 : TMEM_COLS_USED <= 128 ? 128 : TMEM_COLS_USED <= 256 ? 256 : 512;
    static_assert(TMEM_COLS_USED <= 512, "TMEM budget exceeded");
    static_assert(TOTAL <= 227 * 1024, "shared memory budget exceeded");
    static_assert(SW % 2 == 0 && SA % 2 == 0, "ring sizes must be multiples of the number of converter groups");
};

// Position in a CTA's range: linear k-block index `pos` = tile * k_iters + kb.
struct Walk {
    int64_t pos, end, tile;
    int kb, k_iters, m_tiles;
    int n0, m0;
    int64_t tile_base, tile_step;  // the tile behind position `tile` of the walk is tile_base + tile * tile_step
    __device__ __forceinline__ void locate(int mt) {
        const int64_t actual = tile_base + tile * tile_step;
        const int64_t nt = actual / m_tiles;
        n0 = static_cast<int>(nt) * BN;
        m0 = static_cast<int>(actual - nt * m_tiles) * mt;
    }
    __device__ __forceinline__ Walk(int64_t a, int64_t b, int k_iters_, int m_tiles_, int mt, int64_t base = 0, int64_t step = 1)
        : pos(a), end(b), k_iters(k_iters_), m_tiles(m_tiles_), tile_base(base), tile_step(step) {
        tile = a / k_iters_;
        kb = static_cast<int>(a - tile * k_iters_);
        locate(mt);
    }
    __device__ __forceinline__ bool done() const { return pos >= end; }
    __device__ __forceinline__ bool seg_last() const { return kb == k_iters - 1 || pos == end - 1; }
    __device__ __forceinline__ void next(int mt) {
        pos++;
        if (++kb == k_iters) {
            kb = 0;
            tile++;
            locate(mt);
        }
    }
};

__device__ __forceinline__ unsigned long long ld_acquire_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.acquire.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.release.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
// Named barrier 1 belongs to the four epilogue warps (128 threads).
__device__ __forceinline__ void epilogue_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }
// Barrier + OR over the epilogue threads: every thread gets the same answer, so that decisions that depend on a
// flag another warp may raise at any moment (the abort flag, an expired wait) are taken by all 128 threads alike.
__device__ __forceinline__ bool epilogue_any(bool x) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.u32 p, %1, 0;\n\t"
        "bar.red.or.pred q, 1, 128, p;\n\t"
        "selp.u32 %0, 1, 0, q;\n\t}"
        : "=r"(r)
        : "r"(x ? 1u : 0u)
        : "memory");
    return r != 0;
}

__device__ long long g_stream_dbg[32];
__device__ __forceinline__ long long gtime() { long long t; asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t)); return t; }
#define DBG(i) do { if (blockIdx.x == 0) g_stream_dbg[i] = gtime(); } while (0)

template <int MT, int SW, int SA>
__global__ void __launch_bounds__(STREAM_THREADS, 1) tc_stream_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmA,
                                                                      StreamParams p) {
    using L = StreamSmem<MT, SW, SA>;
    constexpr int G = 2;  // converter groups
    if (threadIdx.x == 0) DBG(0);
    dep_trigger();
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFFSET;
    auto w_full = [&](int s) { return bars + 8u * s; };
    auto w_empty = [&](int s) { return bars + 8u * (SW + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * SW + s); };
    auto conv_bar = [&](int s) { return bars + 8u * (2 * SW + SA + s); };
    auto mma_done = [&](int s) { return bars + 8u * (2 * SW + 2 * SA + s); };
    const uint32_t acc_full = bars + 8u * (2 * SW + 3 * SA), acc_empty = acc_full + 8u;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::BAR_OFFSET + 8 * L::N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFFSET + 8 * L::N_BARS + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t cta = blockIdx.x, ctas = gridDim.x;
    // strided: positions 0 .. n_local - 1 of this CTA's walk are tiles cta, cta + ctas, ...
    const int64_t tile_base = p.strided ? cta : 0, tile_step = p.strided ? ctas : 1;
    const int64_t range_a = p.strided ? 0 : (p.units * cta / ctas) * p.gran;
    const int64_t range_b = p.strided ? ((p.units - cta + ctas - 1) / ctas) * p.k_iters : (p.units * (cta + 1) / ctas) * p.gran;
    const int n_iters = static_cast<int>(range_b - range_a);

    if (threadIdx.x == 0) {
        for (int s = 0; s < SW; s++) {
            mbar_init(w_full(s), 1);
            mbar_init(w_empty(s), 128);
        }
        for (int s = 0; s < SA; s++) {
            mbar_init(a_full(s), 1);
            mbar_init(conv_bar(s), 128);
            mbar_init(mma_done(s), 1);
        }
        mbar_init(acc_full, 1);
        mbar_init(acc_empty, 128);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // the first loads go out before the CTA-wide sync; weights that nothing in flight writes even before the previous
        // kernel of the stream has finished, the activations (which that kernel may be producing) only after it
        if (!p.w_static) dep_wait();
        {
            Walk w(range_a, range_b, p.k_iters, p.m_tiles, MT, tile_base, tile_step);
            for (int it = 0; !w.done() && it < SW; w.next(MT), it++) {
                mbar_expect_tx(w_full(it), L::W_BYTES);
                tma_load_2d(base + it * L::W_BYTES, &tmW, w.n0, w.kb * BK, w_full(it));
            }
        }
        DBG(1);
        if (p.w_static) dep_wait();
        DBG(2);
        {
            Walk w(range_a, range_b, p.k_iters, p.m_tiles, MT, tile_base, tile_step);
            for (int it = 0; !w.done() && it < SA; w.next(MT), it++) {
                mbar_expect_tx(a_full(it), L::A_BYTES);
                tma_load_2d(base + L::A_OFFSET + it * L::A_STAGE_BYTES, &tmA, w.kb * BK, w.m0, a_full(it));
            }
        }
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)), "r"(L::TMEM_COLS) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    dep_wait();  // every thread: nothing below reads or writes global memory before the previous grid is complete
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0) DBG(3);
    // TMEM columns: accumulators [0, MT) hi x hi, [MT, 2 MT) hi x lo + lo x hi; weight stage s: hi at 2 MT + 64 s, lo 32 further
    auto whi_col = [&](int s) { return static_cast<uint32_t>(2 * MT + 64 * s); };

    if (warp == 0) {
        // ---------------- weight producer ----------------
        if (lane == 0) {
            Walk w(range_a, range_b, p.k_iters, p.m_tiles, MT, tile_base, tile_step);
            int it = 0;
            for (; !w.done() && it < SW; w.next(MT), it++) {}  // issued before the sync
            for (; !w.done(); w.next(MT), it++) {
                const int s = it % SW;
                if (!mbar_wait(w_empty(s), ((it / SW) - 1) & 1, abort_flag, p.status)) break;
                mbar_expect_tx(w_full(s), L::W_BYTES);
                tma_load_2d(base + s * L::W_BYTES, &tmW, w.n0, w.kb * BK, w_full(s));
            }
        }
    } else if (warp == 2) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            Walk w(range_a, range_b, p.k_iters, p.m_tiles, MT, tile_base, tile_step);
            int it = 0;
            for (; !w.done() && it < SA; w.next(MT), it++) {}
            for (; !w.done(); w.next(MT), it++) {
                const int s = it % SA;
                if (!mbar_wait(mma_done(s), ((it / SA) - 1) & 1, abort_flag, p.status)) break;
                mbar_expect_tx(a_full(s), L::A_BYTES);
                tma_load_2d(base + L::A_OFFSET + s * L::A_STAGE_BYTES, &tmA, w.kb * BK, w.m0, a_full(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D fp32; A (weights, from TMEM) and B (activations, smem) tf32, both K-major; M = 128, N = MT
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((MT >> 3) << 17) | ((BN >> 4) << 24);
            constexpr uint32_t idesc_wide = (1u << 4) | (2u << 7) | (2u << 10) | (((2 * MT) >> 3) << 17) | ((BN >> 4) << 24);
            Walk w(range_a, range_b, p.k_iters, p.m_tiles, MT, tile_base, tile_step);
            int seg = -1;
            for (int it = 0; !w.done(); w.next(MT), it++) {
                const bool first = (w.pos == range_a) || w.kb == 0;
                if (first) {
                    seg++;
                    if (seg >= 1) {  // the epilogue of the previous segment must have pulled the accumulators out
                        if (!mbar_wait(acc_empty, (seg - 1) & 1, abort_flag, p.status)) break;
                        tc_fence_after();
                    }
                }
                const int s = it % SA;
                if (!mbar_wait(conv_bar(s), (it / SA) & 1, abort_flag, p.status)) break;
                if (it == 0) DBG(4);
                if (it == 8) DBG(5);
                if (it == 40) DBG(6);
                tc_fence_after();
                const uint32_t a_hi = base + L::A_OFFSET + s * L::A_STAGE_BYTES;
                const uint32_t w_hi = tmem_base + whi_col(s), w_lo = w_hi + 32;
                const uint32_t d_lo = tmem_base + ((p.mma_mode & 1) ? MT : 0);
                if (p.mma_mode & 2) {
#pragma unroll
                    for (int kk = 0; kk < BK / 8; kk++)
                        tc_mma_tf32_ts(tmem_base, w_hi + kk * 8, smem_desc_k128(a_hi + kk * 32), idesc_wide, (first && kk == 0) ? 0u : 1u);
#pragma unroll
                    for (int kk = 0; kk < BK / 8; kk++) tc_mma_tf32_ts(d_lo, w_lo + kk * 8, smem_desc_k128(a_hi + kk * 32), idesc, 1u);
                } else {
#pragma unroll
                    for (int kk = 0; kk < BK / 8; kk++) {
                        // the lo tile follows the raw tile in shared memory: one descriptor with N = 2 MT covers [hi; lo]
                        const uint64_t da_hi = smem_desc_k128(a_hi + kk * 32);
                        tc_mma_tf32_ts(tmem_base, w_hi + kk * 8, da_hi, idesc_wide, (first && kk == 0) ? 0u : 1u);
                        tc_mma_tf32_ts(d_lo, w_lo + kk * 8, da_hi, idesc, 1u);
                    }
                }
                tc_commit(mma_done(s));
                if (w.seg_last()) { tc_commit(acc_full); DBG(7); }
            }
        }
    } else if (warp >= 4 && warp < 12) {
        // ---------------- converters ----------------
        const int cg = (warp - 4) >> 2;             // converter group 0 .. G-1
        const int t = threadIdx.x - 128 - 128 * cg; // 0..127 inside the group
        const int sub = warp & 3;                   // TMEM sub-partition (32 lanes) this warp owns
        const uint32_t lane_field = static_cast<uint32_t>(sub * 32) << 16;
        for (int it = cg; it < n_iters; it += G) {
            const int sw = it % SW, sa = it % SA;
            if (!(mbar_wait(a_full(sa), (it / SA) & 1, abort_flag, p.status) && mbar_wait(w_full(sw), (it / SW) & 1, abort_flag, p.status))) break;
            const float* wcol = reinterpret_cast<const float*>(base_ptr + sw * L::W_BYTES) + sub * 32 + lane;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    const float x = wcol[(half * 16 + j) * BN];
                    hi[j] = __float_as_uint(x);
                    lo[j] = __float_as_uint(x - __uint_as_float(hi[j] & TF32_MASK));
                }
                tmem_st_x16(tmem_base + lane_field + whi_col(sa) + half * 16, hi);
                tmem_st_x16(tmem_base + lane_field + whi_col(sa) + 32 + half * 16, lo);
            }
            mbar_arrive(w_empty(sw));
            uint8_t* ahi = base_ptr + L::A_OFFSET + sa * L::A_STAGE_BYTES;
            uint8_t* alo = ahi + L::A_BYTES;
#pragma unroll 2
            for (int c = t; c < static_cast<int>(L::A_BYTES / 16); c += 128) {
                const float4 v = *reinterpret_cast<const float4*>(ahi + 16 * c);
                uint4 l;
                l.x = __float_as_uint(v.x - __uint_as_float(__float_as_uint(v.x) & TF32_MASK));
                l.y = __float_as_uint(v.y - __uint_as_float(__float_as_uint(v.y) & TF32_MASK));
                l.z = __float_as_uint(v.z - __uint_as_float(__float_as_uint(v.z) & TF32_MASK));
                l.w = __float_as_uint(v.w - __uint_as_float(__float_as_uint(v.w) & TF32_MASK));
                *reinterpret_cast<uint4*>(alo + 16 * c) = l;
            }
            asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
            fence_proxy_async();
            tc_fence_before();
            mbar_arrive(conv_bar(sa));
        }
    } else if (warp >= 12) {
        // ---------------- epilogue ----------------
        const int sub = warp & 3;
        const int et = threadIdx.x - 384;  // 0..127
        const uint32_t lane_field = static_cast<uint32_t>(sub * 32) << 16;
        const int nl = sub * 32 + lane;    // column inside the tile = TMEM lane
        // CTA that owns linear k-block x (only meaningful when gran == 1)
        auto owner = [&](int64_t x) { return ((x + 1) * ctas - 1) / p.units; };
        auto slot_of = [&](int64_t c, int64_t tile) {  // slot of CTA c's partial of `tile`: 0 if it is c's first tile, else 1
            const int64_t first_tile = (p.units * c / ctas) / p.k_iters;
            return 2 * c + (first_tile == tile ? 0 : 1);
        };
        int64_t part_tile[2] = {-1, -1};
        int n_part = 0;
        bool ok = true;
        int seg = 0;
        int64_t pos = range_a;
        while (pos < range_b && ok) {
            const int64_t tpos = pos / p.k_iters;
            const int kb0 = static_cast<int>(pos - tpos * p.k_iters);
            const int64_t tile = tile_base + tpos * tile_step;
            int64_t len = p.k_iters - kb0;
            if (len > range_b - pos) len = range_b - pos;
            const bool whole = (kb0 == 0 && len == p.k_iters);
            pos += len;
            const int64_t nt = tile / p.m_tiles;
            const int n0 = static_cast<int>(nt) * BN, m0 = static_cast<int>(tile - nt * p.m_tiles) * MT;
            ok = !epilogue_any(!mbar_wait_parked(acc_full, seg & 1, abort_flag, p.status));
            if (!ok) break;
            if (et == 0) DBG(8);
            tc_fence_after();
            const int64_t my_slot = whole ? 0 : slot_of(cta, tile);
            float* slot = p.slots + my_slot * (MT * BN);
            auto store32 = [&](int c0, const float (&v)[32]) {
                if (whole) {
#pragma unroll
                    for (int j = 0; j < 32; j++) {
                        const int64_t m = m0 + c0 + j;
                        if (m < p.M) {
                            p.out[m * p.ldc + n0 + nl] = v[j];
                            for (int d = 0; d < p.n_peer; d++) p.peer_out[d][m * p.ldc + n0 + nl] = v[j];
                        }
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 32; j++) slot[(c0 + j) * BN + nl] = v[j];
                }
            };
            auto load32 = [&](int c0, float (&v)[32]) {  // hi x hi block + (hi x lo + lo x hi) block
                uint32_t r[32], q[32];
                tmem_ld_x32(tmem_base + lane_field + static_cast<uint32_t>(c0), r);
                tmem_ld_x32(tmem_base + lane_field + static_cast<uint32_t>(MT + c0), q);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = __uint_as_float(r[j]) + __uint_as_float(q[j]);
            };
            if constexpr (MT == 64) {
                // everything into registers first, the TMEM block goes back to the MMA thread, then the stores
                float v0[32], v1[32];
                load32(0, v0);
                load32(32, v1);
                tc_fence_before();
                mbar_arrive(acc_empty);
                store32(0, v0);
                store32(32, v1);
            } else {
#pragma unroll
                for (int c0 = 0; c0 < MT; c0 += 32) {
                    float v[32];
                    load32(c0, v);
                    if (c0 + 32 >= MT) {  // the last columns have been read: the next segment's MMAs may overwrite the block
                        tc_fence_before();
                        mbar_arrive(acc_empty);
                    }
                    store32(c0, v);
                }
            }
            if (!whole) {
                // publish: the partial tile is complete in the slot, every member of the tile's group gets a flag
                const int64_t g0 = owner(tile * p.k_iters), g1 = owner(tile * p.k_iters + p.k_iters - 1);
                const int members = static_cast<int>(g1 - g0 + 1);
                __threadfence();
                epilogue_barrier();
                if (members > STREAM_MAX_GROUP) {
                    if (et == 0) {
                        *abort_flag = 1;
                        if (p.status) atomicExch(p.status, RMLK_ERR_INTERNAL);
                    }
                    ok = false;
                    break;
                }
                if (et < members) st_release_u64(p.flags + my_slot * STREAM_MAX_GROUP + et, p.token);
                if (n_part < 2) part_tile[n_part++] = tile;
            }
            seg++;
        }
        // ---------------- fix-up of the tiles this CTA shares with others ----------------
        for (int i = 0; i < n_part && ok; i++) {
            if (epilogue_any(*abort_flag != 0)) break;
            const int64_t tile = part_tile[i];
            const int64_t g0 = owner(tile * p.k_iters), g1 = owner(tile * p.k_iters + p.k_iters - 1);
            const int members = static_cast<int>(g1 - g0 + 1), rank = static_cast<int>(cta - g0);
            // thread j < members waits for member j's flag addressed to this CTA
            if (et < members) {
                const unsigned long long* f = p.flags + slot_of(g0 + et, tile) * STREAM_MAX_GROUP + rank;
                bool seen = false;
                for (uint32_t spin = 0; spin < SPIN_LIMIT; spin++) {
                    if (ld_acquire_u64(f) == p.token) {
                        seen = true;
                        break;
                    }
                    if (*abort_flag) break;
                    __nanosleep(100);
                }
                if (!seen) {
                    *abort_flag = 1;
                    if (p.status) atomicExch(p.status, RMLK_ERR_TIMEOUT);
                }
            }
            __threadfence();
            if (epilogue_any(*abort_flag != 0)) break;
            const int64_t nt = tile / p.m_tiles;
            const int n0 = static_cast<int>(nt) * BN, m0 = static_cast<int>(tile - nt * p.m_tiles) * MT;
            int rows = MT;
            if (p.M - m0 < rows) rows = static_cast<int>(p.M - m0);
            const int c4 = et & 31;
            for (int j = et >> 5;; j += 4) {
                const int m = rank + members * j;  // this member's rows: m % members == rank
                if (m >= rows) break;
                float4 sum = make_float4(0.f, 0.f, 0.f, 0.f);
                for (int q0 = 0; q0 < members; q0 += 4) {
                    float4 v[4];
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        v[u] = make_float4(0.f, 0.f, 0.f, 0.f);
                        if (q0 + u < members)
                            v[u] = __ldcg(reinterpret_cast<const float4*>(p.slots + slot_of(g0 + q0 + u, tile) * (MT * BN) + m * BN) + c4);
                    }
#pragma unroll
                    for (int u = 0; u < 4; u++) {
                        if (q0 + u < members) {
                            sum.x += v[u].x;
                            sum.y += v[u].y;
                            sum.z += v[u].z;
                            sum.w += v[u].w;
                        }
                    }
                }
                const int64_t at = static_cast<int64_t>(m0 + m) * p.ldc + n0 + 4 * c4;
                *reinterpret_cast<float4*>(p.out + at) = sum;
                for (int d = 0; d < p.n_peer; d++) *reinterpret_cast<float4*>(p.peer_out[d] + at) = sum;
            }
            // the flags addressed to this CTA have served: clear them for the next launch that uses this scratch
            epilogue_barrier();
            if (et < members) p.flags[slot_of(g0 + et, tile) * STREAM_MAX_GROUP + rank] = 0ull;
        }
    }
    if (threadIdx.x == 384) DBG(9);
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0) DBG(10);
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

}  // namespace tc
}  // namespace rmlk
