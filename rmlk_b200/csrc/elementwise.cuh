// Broadcast elementwise engine shared by the binary / pow / unary / cast / where / expand launchers.
//
// Host side: the (shape, per-operand strides) description is *stride-collapsed* — size-1 dims are
// dropped and neighbouring dims are merged whenever every operand walks them as one dense run (or
// broadcasts both) — so that the common cases of the reference's op graphs
// (same-shape, tensor∘scalar, [.., N]∘[N], [.., N]∘[.., 1], [B,H,S,D]∘[1,1,S,D]) end up with rank 1–2.
//
// Device side, two kernels:
//   ew_vec_kernel    the innermost collapsed dim is walked in packs of E elements (E chosen so the
//                    narrowest operand still moves 16 bytes per access); each operand is either dense
//                    along it (128-bit loads) or broadcast along it (one scalar load, splat).  Outer
//                    coordinates are decoded once per pack with 32-bit multiply-high division.
//   ew_scalar_kernel any strides, one element per thread-iteration; also serves ragged tails and
//                    tensors too large for 32-bit item indices (WIDE).
#pragma once

#include "common.cuh"

namespace rmlk {

constexpr int EW_MAX_OUTER = RMLK_MAX_RANK;  // outer dims after collapse (inner dim held apart)
constexpr uint64_t EW_NARROW_LIMIT = (1ull << 31) - 1;

template <int NIN>
struct EwParams {
    int outer_rank;
    uint64_t inner_items;           // packs (vec) or elements (scalar) along the inner dim
    uint64_t n_items;               // total items = prod(outer) * inner_items
    FastDiv inner_div;              // divides by inner_items
    FastDiv div[EW_MAX_OUTER];      // outer dims, innermost-outer first
    uint64_t wide_dim[EW_MAX_OUTER];
    int64_t ostride[NIN][EW_MAX_OUTER];
    int64_t istride[NIN];           // element stride along the inner dim (vec: 0 or 1)
};

template <int NIN>
struct EwDesc {
    int rank;  // >= 1
    int64_t shape[RMLK_MAX_RANK];
    int64_t strides[NIN][RMLK_MAX_RANK];
    int64_t n;
};

// Collapse (shape, strides) → EwDesc.  Output is dense row-major over `shape`.
template <int NIN>
inline EwDesc<NIN> ew_collapse(int rank, const int64_t* shape, const int64_t* const* strides) {
    EwDesc<NIN> d;
    d.rank = 0;
    d.n = 1;
    for (int i = 0; i < rank; i++) d.n *= shape[i];
    for (int i = 0; i < rank; i++) {
        if (shape[i] == 1) continue;
        int64_t st[NIN];
        for (int k = 0; k < NIN; k++) st[k] = strides[k][i];
        if (d.rank > 0) {
            // try to merge dim i into the previous kept dim: prev_stride == this_stride * this_shape
            bool ok = true;
            for (int k = 0; k < NIN; k++)
                if (d.strides[k][d.rank - 1] != st[k] * shape[i]) ok = false;
            if (ok) {
                d.shape[d.rank - 1] *= shape[i];
                for (int k = 0; k < NIN; k++) d.strides[k][d.rank - 1] = st[k];
                continue;
            }
        }
        d.shape[d.rank] = shape[i];
        for (int k = 0; k < NIN; k++) d.strides[k][d.rank] = st[k];
        d.rank++;
    }
    if (d.rank == 0) {
        d.rank = 1;
        d.shape[0] = 1;
        for (int k = 0; k < NIN; k++) d.strides[k][0] = 1;
    }
    return d;
}

template <int NIN>
inline EwParams<NIN> ew_params(const EwDesc<NIN>& d, int E) {
    EwParams<NIN> p;
    p.outer_rank = d.rank - 1;
    const int64_t inner = d.shape[d.rank - 1];
    p.inner_items = static_cast<uint64_t>(inner / E);
    p.inner_div = FastDiv(p.inner_items && p.inner_items <= EW_NARROW_LIMIT ? static_cast<uint32_t>(p.inner_items) : 1);
    uint64_t items = p.inner_items;
    for (int j = 0; j < p.outer_rank; j++) {
        const int dim = d.rank - 2 - j;
        p.div[j] = FastDiv(static_cast<uint32_t>(d.shape[dim]));
        p.wide_dim[j] = static_cast<uint64_t>(d.shape[dim]);
        items *= static_cast<uint64_t>(d.shape[dim]);
        for (int k = 0; k < NIN; k++) p.ostride[k][j] = d.strides[k][dim];
    }
    p.n_items = items;
    for (int k = 0; k < NIN; k++) p.istride[k] = d.strides[k][d.rank - 1];
    return p;
}

// Elements per pack: the narrowest operand moves 16 bytes, the widest at most 64.
template <typename... Ts>
struct EwPack {
    static constexpr size_t mn = [] { size_t m = 16; ((m = sizeof(Ts) < m ? sizeof(Ts) : m), ...); return m; }();
    static constexpr size_t mx = [] { size_t m = 1; ((m = sizeof(Ts) > m ? sizeof(Ts) : m), ...); return m; }();
    static constexpr int E = static_cast<int>((16 / mn) < (64 / mx) ? (16 / mn) : (64 / mx));
};

template <int NIN, bool WIDE>
__device__ __forceinline__ void ew_decode(const EwParams<NIN>& p, uint64_t item, uint64_t& inner_i, int64_t (&off)[NIN]) {
#pragma unroll
    for (int k = 0; k < NIN; k++) off[k] = 0;
    if (p.outer_rank == 0) {
        inner_i = item;
        return;
    }
    if constexpr (!WIDE) {
        uint32_t o, ii;
        p.inner_div.divmod(static_cast<uint32_t>(item), o, ii);
        inner_i = ii;
#pragma unroll
        for (int j = 0; j < EW_MAX_OUTER; j++) {
            if (j >= p.outer_rank) break;
            uint32_t q, c;
            p.div[j].divmod(o, q, c);
            o = q;
#pragma unroll
            for (int k = 0; k < NIN; k++) off[k] += static_cast<int64_t>(c) * p.ostride[k][j];
        }
    } else {
        uint64_t o = item / p.inner_items;
        inner_i = item - o * p.inner_items;
        for (int j = 0; j < p.outer_rank; j++) {
            const uint64_t q = o / p.wide_dim[j];
            const uint64_t c = o - q * p.wide_dim[j];
            o = q;
#pragma unroll
            for (int k = 0; k < NIN; k++) off[k] += static_cast<int64_t>(c) * p.ostride[k][j];
        }
    }
}

template <typename T, int E>
__device__ __forceinline__ Pack<T, E> ew_load(const T* base, int64_t off, uint64_t inner_i, int64_t istride) {
    if (istride != 0) return load_pack<T, E>(base + off + static_cast<int64_t>(inner_i) * E);
    Pack<T, E> r;
    const T s = base[off];
#pragma unroll
    for (int e = 0; e < E; e++) r.v[e] = s;
    return r;
}

constexpr int EW_BLOCK = 256;

// ---- one input ------------------------------------------------------------------------------
template <int E, typename F, typename TO, typename T0>
__global__ void __launch_bounds__(EW_BLOCK) ew_vec_kernel1(EwParams<1> p, TO* __restrict__ out, const T0* __restrict__ a) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[1];
    ew_decode<1, false>(p, item, ii, off);
    const Pack<T0, E> va = ew_load<T0, E>(a, off[0], ii, p.istride[0]);
    Pack<TO, E> r;
#pragma unroll
    for (int e = 0; e < E; e++) r.v[e] = F::apply(va.v[e]);
    store_pack<TO, E>(out + item * E, r);
}

template <bool WIDE, typename F, typename TO, typename T0>
__global__ void __launch_bounds__(EW_BLOCK) ew_scalar_kernel1(EwParams<1> p, TO* __restrict__ out, const T0* __restrict__ a) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[1];
    ew_decode<1, WIDE>(p, item, ii, off);
    out[item] = F::apply(a[off[0] + static_cast<int64_t>(ii) * p.istride[0]]);
}

// ---- two inputs -----------------------------------------------------------------------------
template <int E, typename F, typename TO, typename T0, typename T1>
__global__ void __launch_bounds__(EW_BLOCK)
    ew_vec_kernel2(EwParams<2> p, TO* __restrict__ out, const T0* __restrict__ a, const T1* __restrict__ b) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[2];
    ew_decode<2, false>(p, item, ii, off);
    const Pack<T0, E> va = ew_load<T0, E>(a, off[0], ii, p.istride[0]);
    const Pack<T1, E> vb = ew_load<T1, E>(b, off[1], ii, p.istride[1]);
    Pack<TO, E> r;
#pragma unroll
    for (int e = 0; e < E; e++) r.v[e] = F::apply(va.v[e], vb.v[e]);
    store_pack<TO, E>(out + item * E, r);
}

template <bool WIDE, typename F, typename TO, typename T0, typename T1>
__global__ void __launch_bounds__(EW_BLOCK)
    ew_scalar_kernel2(EwParams<2> p, TO* __restrict__ out, const T0* __restrict__ a, const T1* __restrict__ b) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[2];
    ew_decode<2, WIDE>(p, item, ii, off);
    out[item] = F::apply(a[off[0] + static_cast<int64_t>(ii) * p.istride[0]],
                         b[off[1] + static_cast<int64_t>(ii) * p.istride[1]]);
}

// ---- three inputs ---------------------------------------------------------------------------
template <int E, typename F, typename TO, typename T0, typename T1, typename T2>
__global__ void __launch_bounds__(EW_BLOCK) ew_vec_kernel3(EwParams<3> p, TO* __restrict__ out, const T0* __restrict__ a,
                                                           const T1* __restrict__ b, const T2* __restrict__ c) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[3];
    ew_decode<3, false>(p, item, ii, off);
    const Pack<T0, E> va = ew_load<T0, E>(a, off[0], ii, p.istride[0]);
    const Pack<T1, E> vb = ew_load<T1, E>(b, off[1], ii, p.istride[1]);
    const Pack<T2, E> vc = ew_load<T2, E>(c, off[2], ii, p.istride[2]);
    Pack<TO, E> r;
#pragma unroll
    for (int e = 0; e < E; e++) r.v[e] = F::apply(va.v[e], vb.v[e], vc.v[e]);
    store_pack<TO, E>(out + item * E, r);
}

template <bool WIDE, typename F, typename TO, typename T0, typename T1, typename T2>
__global__ void __launch_bounds__(EW_BLOCK) ew_scalar_kernel3(EwParams<3> p, TO* __restrict__ out, const T0* __restrict__ a,
                                                              const T1* __restrict__ b, const T2* __restrict__ c) {
    dep_sync();
    const uint64_t item = static_cast<uint64_t>(blockIdx.x) * EW_BLOCK + threadIdx.x;
    if (item >= p.n_items) return;
    uint64_t ii;
    int64_t off[3];
    ew_decode<3, WIDE>(p, item, ii, off);
    out[item] = F::apply(a[off[0] + static_cast<int64_t>(ii) * p.istride[0]],
                         b[off[1] + static_cast<int64_t>(ii) * p.istride[1]],
                         c[off[2] + static_cast<int64_t>(ii) * p.istride[2]]);
}

// ---------------------------------------------------------------------------------------------
// host dispatch
// ---------------------------------------------------------------------------------------------
inline int ew_validate(int rank, const int64_t* shape) {
    if (rank < 0 || rank > RMLK_MAX_RANK) return fail(RMLK_ERR_INVALID_ARG, "rank must be in [0, 8]");
    if (rank > 0 && !shape) return fail(RMLK_ERR_INVALID_ARG, "shape is NULL");
    for (int i = 0; i < rank; i++)
        if (shape[i] < 0) return fail(RMLK_ERR_INVALID_ARG, "negative dimension");
    return RMLK_OK;
}

template <int NIN>
inline bool ew_vec_ok(const EwDesc<NIN>& d, int E, const size_t* elem_sizes /*NIN*/, const void* const* ptrs /*NIN*/,
                      const void* out, size_t out_size) {
    if (E <= 1) return false;
    const int64_t inner = d.shape[d.rank - 1];
    if (d.rank > 1 && inner % E != 0) return false;
    if (d.rank == 1 && inner < E) return false;
    auto need = [&](size_t sz) { return (sz * E) >= 16 ? size_t(16) : sz * E; };
    if (!aligned_to(out, need(out_size))) return false;
    for (int k = 0; k < NIN; k++) {
        const int64_t is = d.strides[k][d.rank - 1];
        if (is != 0 && is != 1) return false;
        if (is == 1) {
            if (!aligned_to(ptrs[k], need(elem_sizes[k]))) return false;
            for (int j = 0; j < d.rank - 1; j++)
                if (d.strides[k][j] % E != 0) return false;
        }
    }
    return true;
}

#define EW_GRID(items) static_cast<unsigned>(((items) + EW_BLOCK - 1) / EW_BLOCK)

// The three launchers share one shape: try the vector kernel on the E-divisible part, finish (or
// fall back) with the scalar kernel.
template <typename F, typename TO, typename T0>
int ew_launch1(cudaStream_t st, int rank, const int64_t* shape, const int64_t* s0, const T0* a, TO* out) {
    const int64_t* strides[1] = {s0};
    EwDesc<1> d = ew_collapse<1>(rank, shape, strides);
    if (d.n == 0) return RMLK_OK;
    constexpr int E = EwPack<TO, T0>::E;
    const size_t sizes[1] = {sizeof(T0)};
    const void* ptrs[1] = {a};
    int64_t done = 0;
    if (ew_vec_ok<1>(d, E, sizes, ptrs, out, sizeof(TO))) {
        EwDesc<1> dv = d;
        if (d.rank == 1) dv.shape[0] = d.shape[0] - d.shape[0] % E;
        EwParams<1> p = ew_params<1>(dv, E);
        if (p.n_items <= EW_NARROW_LIMIT) {
            launch_dep(ew_vec_kernel1<E, F, TO, T0>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out, a);
            RMLK_CHECK_LAUNCH("ew_vec_kernel1");
            if (d.rank > 1 || dv.shape[0] == d.shape[0]) return RMLK_OK;
            done = dv.shape[0];
        }
    }
    EwDesc<1> ds = d;
    const T0* a2 = a;
    if (done) {  // rank-1 tail
        ds.shape[0] = d.shape[0] - done;
        a2 = a + done * d.strides[0][0];
    }
    EwParams<1> p = ew_params<1>(ds, 1);
    if (p.n_items <= EW_NARROW_LIMIT)
        launch_dep(ew_scalar_kernel1<false, F, TO, T0>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2);
    else
        launch_dep(ew_scalar_kernel1<true, F, TO, T0>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2);
    RMLK_CHECK_LAUNCH("ew_scalar_kernel1");
    return RMLK_OK;
}

template <typename F, typename TO, typename T0, typename T1>
int ew_launch2(cudaStream_t st, int rank, const int64_t* shape, const int64_t* s0, const int64_t* s1, const T0* a,
               const T1* b, TO* out) {
    const int64_t* strides[2] = {s0, s1};
    EwDesc<2> d = ew_collapse<2>(rank, shape, strides);
    if (d.n == 0) return RMLK_OK;
    constexpr int E = EwPack<TO, T0, T1>::E;
    const size_t sizes[2] = {sizeof(T0), sizeof(T1)};
    const void* ptrs[2] = {a, b};
    int64_t done = 0;
    if (ew_vec_ok<2>(d, E, sizes, ptrs, out, sizeof(TO))) {
        EwDesc<2> dv = d;
        if (d.rank == 1) dv.shape[0] = d.shape[0] - d.shape[0] % E;
        EwParams<2> p = ew_params<2>(dv, E);
        if (p.n_items <= EW_NARROW_LIMIT) {
            launch_dep(ew_vec_kernel2<E, F, TO, T0, T1>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out, a, b);
            RMLK_CHECK_LAUNCH("ew_vec_kernel2");
            if (d.rank > 1 || dv.shape[0] == d.shape[0]) return RMLK_OK;
            done = dv.shape[0];
        }
    }
    EwDesc<2> ds = d;
    const T0* a2 = a;
    const T1* b2 = b;
    if (done) {
        ds.shape[0] = d.shape[0] - done;
        a2 = a + done * d.strides[0][0];
        b2 = b + done * d.strides[1][0];
    }
    EwParams<2> p = ew_params<2>(ds, 1);
    if (p.n_items <= EW_NARROW_LIMIT)
        launch_dep(ew_scalar_kernel2<false, F, TO, T0, T1>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2, b2);
    else
        launch_dep(ew_scalar_kernel2<true, F, TO, T0, T1>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2, b2);
    RMLK_CHECK_LAUNCH("ew_scalar_kernel2");
    return RMLK_OK;
}

template <typename F, typename TO, typename T0, typename T1, typename T2>
int ew_launch3(cudaStream_t st, int rank, const int64_t* shape, const int64_t* s0, const int64_t* s1,
               const int64_t* s2, const T0* a, const T1* b, const T2* c, TO* out) {
    const int64_t* strides[3] = {s0, s1, s2};
    EwDesc<3> d = ew_collapse<3>(rank, shape, strides);
    if (d.n == 0) return RMLK_OK;
    constexpr int E = EwPack<TO, T0, T1, T2>::E;
    const size_t sizes[3] = {sizeof(T0), sizeof(T1), sizeof(T2)};
    const void* ptrs[3] = {a, b, c};
    int64_t done = 0;
    if (ew_vec_ok<3>(d, E, sizes, ptrs, out, sizeof(TO))) {
        EwDesc<3> dv = d;
        if (d.rank == 1) dv.shape[0] = d.shape[0] - d.shape[0] % E;
        EwParams<3> p = ew_params<3>(dv, E);
        if (p.n_items <= EW_NARROW_LIMIT) {
            launch_dep(ew_vec_kernel3<E, F, TO, T0, T1, T2>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out, a, b, c);
            RMLK_CHECK_LAUNCH("ew_vec_kernel3");
            if (d.rank > 1 || dv.shape[0] == d.shape[0]) return RMLK_OK;
            done = dv.shape[0];
        }
    }
    EwDesc<3> ds = d;
    const T0* a2 = a;
    const T1* b2 = b;
    const T2* c2 = c;
    if (done) {
        ds.shape[0] = d.shape[0] - done;
        a2 = a + done * d.strides[0][0];
        b2 = b + done * d.strides[1][0];
        c2 = c + done * d.strides[2][0];
    }
    EwParams<3> p = ew_params<3>(ds, 1);
    if (p.n_items <= EW_NARROW_LIMIT)
        launch_dep(ew_scalar_kernel3<false, F, TO, T0, T1, T2>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2, b2, c2);
    else
        launch_dep(ew_scalar_kernel3<true, F, TO, T0, T1, T2>, dim3(EW_GRID(p.n_items)), dim3(EW_BLOCK), 0, st, p, out + done, a2, b2, c2);
    RMLK_CHECK_LAUNCH("ew_scalar_kernel3");
    return RMLK_OK;
}

}  // namespace rmlk
