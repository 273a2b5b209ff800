// tc_gemm_kernel: one CTA computes a [MT x 128] tile of C (optionally one K-split of it).
#pragma once

#include "matmul_tc.cuh"

namespace rmlk {
namespace tc {

template <int MT, int SW, int SA, int G, bool PEERS>
__global__ void __launch_bounds__(threads_for(G), 1) tc_gemm_kernel(const __grid_constant__ CUtensorMap tmW,
                                                              const __grid_constant__ CUtensorMap tmA, TcParams p) {
    using L = SmemLayout<MT, SW, SA>;
    dep_trigger();  // the next kernel of the stream may be scheduled; it waits for this grid before touching memory
    // the G converter groups take k-blocks in turn; a ring slot must always come back to the same group, or a
    // group could be two barrier phases behind and mistake an old phase for the one it waits for
    static_assert(SW % G == 0 && SA % G == 0, "ring sizes must be multiples of the number of converter groups");
    constexpr int A_WARP = 2 + 4 * G;  // the warp after the converters
    extern __shared__ uint8_t smem_raw[];
    const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
    const uint32_t bars = base + L::BAR_OFFSET;
    // 8-byte slots: w_full[SW], w_empty[SW], a_full[SA], conv[SA], mma_done[SA], accum; then the TMEM base slot and
    // the abort flag
    auto w_full = [&](int s) { return bars + 8u * s; };
    auto w_empty = [&](int s) { return bars + 8u * (SW + s); };
    auto a_full = [&](int s) { return bars + 8u * (2 * SW + s); };
    auto conv_bar = [&](int s) { return bars + 8u * (2 * SW + SA + s); };
    auto mma_done = [&](int s) { return bars + 8u * (2 * SW + 2 * SA + s); };
    const uint32_t accum_bar = bars + 8u * (2 * SW + 3 * SA);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(base_ptr + L::BAR_OFFSET + 8 * L::N_BARS);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(base_ptr + L::BAR_OFFSET + 8 * L::N_BARS + 8);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // an activation stage holds two tiles: the lo twin first, then the raw tile (its own hi part)
    constexpr uint32_t raw_off = L::A_BYTES, lo_off = 0u;
    const int n0 = blockIdx.x * BN;
    const int split = blockIdx.y;
    const int m0 = blockIdx.z * MT;
    const int it_begin = split * p.k_iters_per_split;
    int n_iters = p.k_iters_total - it_begin;
    if (n_iters > p.k_iters_per_split) n_iters = p.k_iters_per_split;

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
        mbar_init(accum_bar, 1);
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
        // The first loads need nothing but their barriers: they go out now, while TMEM is being allocated and the
        // other warps arrive, instead of after the CTA-wide sync (the start-up latency of a CTA is a large part of
        // a launch with few k-blocks).  Weights that nothing in flight writes are requested even before the
        // previous kernel of the stream has finished (this grid may have been scheduled early, see dep_wait); the
        // activations, which that kernel may be producing, only after it.
        if (!p.w_static) dep_wait();
        for (int it = 0; it < n_iters && it < SW; it++) {
            mbar_expect_tx(w_full(it), L::W_BYTES);
            tma_load_2d(base + it * L::W_BYTES, &tmW, n0, (it_begin + it) * BK, w_full(it));
        }
        if (p.w_static) dep_wait();
        for (int it = 0; it < n_iters && it < SA; it++) {
            mbar_expect_tx(a_full(it), L::A_BYTES);
            tma_load_2d(base + L::A_OFFSET + it * L::A_STAGE_BYTES + raw_off, &tmA, (it_begin + it) * BK, m0, a_full(it));
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
    // TMEM columns: [0, 2 MT) accumulators (hi*lo + lo*hi | hi*hi); activation stage s: weights hi at 2 MT + 64 s, lo 32 further
    auto whi_col = [&](int s) { return static_cast<uint32_t>(2 * MT + 64 * s); };

    if (warp == 0) {
        // ---------------- weight producer ----------------
        // A weight block leaves shared memory when its converter group has copied it into TMEM, well before the MMAs
        // that use it complete: the ring turns over faster than the activation ring and keeps more of the weight
        // stream in flight.
        if (lane == 0) {
            for (int it = SW; it < n_iters; it++) {  // the first SW loads were issued before the CTA-wide sync
                const int s = it % SW;
                if (!mbar_wait(w_empty(s), ((it / SW) - 1) & 1, abort_flag, p.status)) break;
                mbar_expect_tx(w_full(s), L::W_BYTES);
                tma_load_2d(base + s * L::W_BYTES, &tmW, n0, (it_begin + it) * BK, w_full(s));
            }
        }
    } else if (warp == A_WARP) {
        // ---------------- activation producer ----------------
        if (lane == 0) {
            for (int it = SA; it < n_iters; it++) {
                const int s = it % SA;
                if (!mbar_wait(mma_done(s), ((it / SA) - 1) & 1, abort_flag, p.status)) break;
                mbar_expect_tx(a_full(s), L::A_BYTES);
                tma_load_2d(base + L::A_OFFSET + s * L::A_STAGE_BYTES + raw_off, &tmA, (it_begin + it) * BK, m0, a_full(s));
            }
        }
    } else if (warp == 1) {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            // D fp32; A (weights, from TMEM) and B (activations, smem) tf32, both K-major; M = 128, N = MT
            constexpr uint32_t idesc = (1u << 4) | (2u << 7) | (2u << 10) | ((MT >> 3) << 17) | ((BN >> 4) << 24);
            constexpr uint32_t idesc_wide = (1u << 4) | (2u << 7) | (2u << 10) | (((2 * MT) >> 3) << 17) | ((BN >> 4) << 24);
            // This one thread's instruction stream is close to the critical path (eight MMAs per k-block of 16 KB), so the loop
            // keeps running counters instead of dividing, and builds each operand descriptor with one addition: the upper
            // half of a descriptor is constant and the lower half is the address in 16-byte units.
            const uint64_t desc0 = smem_desc_k128(base + L::A_OFFSET);
            const uint32_t desc_hi = static_cast<uint32_t>(desc0 >> 32), desc_lo0 = static_cast<uint32_t>(desc0);
            uint32_t s = 0, phase = 0;
            for (int it = 0; it < n_iters; it++) {
                if (!mbar_wait(conv_bar(s), phase, abort_flag, p.status)) break;
                tc_fence_after();
                const uint32_t stage_lo = desc_lo0 + s * (L::A_STAGE_BYTES >> 4), raw_lo = stage_lo + (raw_off >> 4);
                const uint32_t w_hi = tmem_base + whi_col(s), w_lo = w_hi + 32;
                // a k-step of 8 is 8 TMEM columns of the weights and 32 bytes inside the swizzled activation rows.
                // One descriptor with N = 2 MT covers both tiles of the stage: W_hi x [first; second] fills accumulator
                // columns [0, MT) and [MT, 2 MT); then W_lo x x_hi goes into [0, MT).  With the lo tile first that block is
                // hi x lo: both small products stay out of the large hi x hi sums (the tensor core truncates when it adds
                // into its fp32 accumulator), which halves the error.
                if (it == 0)
                    tc_mma_tf32_ts(tmem_base, w_hi, smem_desc_k128(base + L::A_OFFSET), idesc_wide, 0u);
                else
                    tc_mma_tf32_ts_acc(tmem_base, w_hi, stage_lo, desc_hi, idesc_wide);
                tc_mma_tf32_ts_acc(tmem_base, w_lo, raw_lo, desc_hi, idesc);
#pragma unroll
                for (int kk = 1; kk < BK / 8; kk++) {
                    tc_mma_tf32_ts_acc(tmem_base, w_hi + kk * 8, stage_lo + kk * 2, desc_hi, idesc_wide);
                    tc_mma_tf32_ts_acc(tmem_base, w_lo + kk * 8, raw_lo + kk * 2, desc_hi, idesc);
                }
                tc_commit(mma_done(s));
                if (++s == SA) {
                    s = 0;
                    phase ^= 1;
                }
            }
            tc_commit(accum_bar);
        }
    } else {
        // ---------------- converters, then epilogue ----------------
        // G converter groups of four warps take the k-blocks in turn, so that the latency of one block's
        // shared-memory reads, TMEM stores and their completion wait overlaps the other groups' work
        const int cg = (warp - 2) >> 2;            // converter group 0 .. G-1
        const int t = threadIdx.x - 64 - 128 * cg; // 0..127 inside the group
        const int sub = warp & 3;                  // TMEM sub-partition (32 lanes) this warp owns
        const uint32_t lane_field = static_cast<uint32_t>(sub * 32) << 16;
        bool ok = true;
        for (int it = cg; it < n_iters && ok; it += G) {
            const int sw = it % SW, sa = it % SA;
            // the activation block of k-block `it` is requested only after the MMAs of k-block it - SA have completed,
            // so its arrival also says that TMEM block sa and the lo twin in shared memory are free again
            ok = mbar_wait(a_full(sa), (it / SA) & 1, abort_flag, p.status) && mbar_wait(w_full(sw), (it / SW) & 1, abort_flag, p.status);
            if (!ok) break;
            // weights: this thread owns column n0 + sub*32 + lane = TMEM lane sub*32 + lane of the [32 k][128 n] block
            // (a warp reads 32 consecutive floats of a row: conflict-free).  32 k values go to TMEM as tf32 hi and lo
            // (16 columns per store)
            const float* wcol = reinterpret_cast<const float*>(base_ptr + sw * L::W_BYTES) + sub * 32 + lane;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                uint32_t hi[16], lo[16];
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    // The MMA reads only the tf32 part of an operand word (sign, exponent, 10 mantissa bits):
                    // the raw fp32 word already is its own truncated `hi`; lo = x - trunc(x) is exact in fp32.
                    const float x = wcol[(half * 16 + j) * BN];
                    hi[j] = __float_as_uint(x);
                    lo[j] = __float_as_uint(x - __uint_as_float(hi[j] & TF32_MASK));
                }
                tmem_st_x16(tmem_base + lane_field + whi_col(sa) + half * 16, hi);
                tmem_st_x16(tmem_base + lane_field + whi_col(sa) + 32 + half * 16, lo);
            }
            mbar_arrive(w_empty(sw));  // this thread's 32 values are in registers / on their way to TMEM: the block may be refilled
            // activations: the tile as loaded is its own hi part; lo goes into the twin tile at the same swizzled offsets
            uint8_t* ahi = base_ptr + L::A_OFFSET + sa * L::A_STAGE_BYTES + raw_off;
            uint8_t* alo = base_ptr + L::A_OFFSET + sa * L::A_STAGE_BYTES + lo_off;
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
        if (ok) ok = mbar_wait(accum_bar, 0, abort_flag, p.status);
        if (ok && !p.cluster_reduce) {
            tc_fence_after();
            const int64_t n = n0 + sub * 32 + lane;
            float* out = p.out + (p.ksplit > 1 ? static_cast<int64_t>(split) * p.M * p.N : 0);
#pragma unroll
            for (int c0 = 32 * cg; c0 < MT; c0 += 32 * G) {
                uint32_t r[32], q[32];
                tmem_ld_x32(tmem_base + lane_field + c0, r);
                tmem_ld_x32(tmem_base + lane_field + MT + c0, q);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int64_t m = m0 + c0 + j;
                    if (m < p.M) {
                        const float v = __uint_as_float(r[j]) + __uint_as_float(q[j]);
                        out[m * p.ldc + n] = v;
                        if constexpr (PEERS)
                            for (int d = 0; d < p.n_peer; d++) p.peer_out[d][m * p.ldc + n] = v;
                    }
                }
            }
        }
    }
    if (p.cluster_reduce) {
        // Split-K inside a thread-block cluster: the ksplit CTAs of a cluster hold the partial sums of one tile.
        // CTA `rank` owns rows [rank * rows_per, (rank + 1) * rows_per) of the tile: every CTA stores that
        // slice of its partial into slot [its own rank] of the owner's shared memory (the pipeline rings, idle
        // by then), and each owner adds its ksplit slots in rank order - a fixed order, so the result does not
        // depend on timing - and writes its rows of C.  No scratch in global memory, no second kernel.
        const uint32_t ks = static_cast<uint32_t>(p.ksplit), rank = cluster_ctarank();
        const uint32_t rows_per = (MT + ks - 1) / ks;
        cluster_sync_all();  // every CTA of the cluster has drained its pipeline: its ring buffers are free
        if (warp >= 2 && warp < A_WARP && !*abort_flag) {
            const int cg = (warp - 2) >> 2, sub = warp & 3;
            const uint32_t lane_field = static_cast<uint32_t>(sub * 32) << 16;
            tc_fence_after();
#pragma unroll
            for (int c0 = 32 * cg; c0 < MT; c0 += 32 * G) {
                uint32_t r[32], q[32];
                tmem_ld_x32(tmem_base + lane_field + c0, r);
                tmem_ld_x32(tmem_base + lane_field + MT + c0, q);
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const uint32_t ml_tile = static_cast<uint32_t>(c0 + j);
                    const uint32_t owner = ml_tile / rows_per, ml = ml_tile - owner * rows_per;
                    const uint32_t local = base + ((rank * rows_per + ml) * BN + sub * 32 + lane) * 4u;
                    st_shared_cluster_f32(mapa_shared(local, owner), __uint_as_float(r[j]) + __uint_as_float(q[j]));
                }
            }
        }
        cluster_sync_all();  // all slices delivered (release / acquire at cluster scope)
        if (warp >= 2 && warp < A_WARP && !*abort_flag) {
            const float* buf = reinterpret_cast<const float*>(base_ptr);
            for (uint32_t idx = threadIdx.x - 64; idx < rows_per * BN; idx += 128 * G) {
                const uint32_t ml = idx / BN, n = idx - ml * BN;
                const uint32_t row = rank * rows_per + ml;
                const int64_t m = m0 + row;
                if (row < static_cast<uint32_t>(MT) && m < p.M) {
                    float s = buf[ml * BN + n];
                    for (uint32_t r2 = 1; r2 < ks; r2++) s += buf[(r2 * rows_per + ml) * BN + n];
                    p.out[m * p.ldc + n0 + n] = s;
                    if constexpr (PEERS)
                        for (int d = 0; d < p.n_peer; d++) p.peer_out[d][m * p.ldc + n0 + n] = s;
                }
            }
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::TMEM_COLS) : "memory");
    }
}

}  // namespace tc
}  // namespace rmlk
