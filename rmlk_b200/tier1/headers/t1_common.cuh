// Symbol-compatible kernels ("tier 1"): the same extern "C" entry-point names and parameter lists as the
// reference's PTX modules (cuda/src/ptx/*.cu), written so that the reference's unmodified launch wrappers
// (cuda/src/kernels/*.rs: grid = ceil(n / 128), block = 128, the `info` buffers its backends upload) get
// correct results from them.  Plain CUDA C++ without sm_100a-only instructions, so the reference's build
// script can compile them to PTX for compute capability 10.0 as it does its own files.
//
// What differs from the reference's bodies, inside that contract:
//  * 64-bit element indices throughout (the reference's `unsigned int` loop counters wrap at 2^32 elements);
//  * the per-element index decode is one loop shared by all operands, in 32-bit arithmetic when the tensor has
//    fewer than 2^32 elements, and stops once the remaining index is zero (the reference divides 64-bit values
//    for every operand and every dim);
//  * ReduceMean decodes an output's base offset once and walks the reduced dims with an odometer instead of
//    re-deriving every coordinate for every element;
//  * Trilu writes zeros to masked elements (the reference leaves them unwritten and relies on fresh memory);
//    ScatterND "none" assigns (the reference computes in + 0 * out, which turns NaN / Inf in the overwritten
//    slot into NaN).
#pragma once

#include <cuda_fp16.h>
#include <stdint.h>

#include <type_traits>

namespace t1 {

constexpr int MAX_RANK = 32;  // the reference's reduce kernel sizes its coordinate arrays for 32 dims

__device__ __forceinline__ size_t global_tid() { return static_cast<size_t>(blockIdx.x) * blockDim.x + threadIdx.x; }
__device__ __forceinline__ size_t grid_threads() { return static_cast<size_t>(blockDim.x) * gridDim.x; }

// Offsets of output element i in up to three operands at once: one row-major decode over dims shared by all of
// them (32-bit arithmetic when the tensor has fewer than 2^32 elements, which a 64-bit divide costs several
// times over), stopping as soon as the remaining index is zero.
template <int NOPS>
__device__ __forceinline__ void offsets_of(size_t i, const size_t* dims, const size_t* const (&strides)[NOPS], int rank, bool small, size_t (&off)[NOPS]) {
#pragma unroll
    for (int o = 0; o < NOPS; o++) off[o] = 0;
    if (small) {
        uint32_t t = static_cast<uint32_t>(i);
        for (int d = rank - 1; d >= 0 && t != 0; d--) {
            const uint32_t n = static_cast<uint32_t>(dims[d]);
            const uint32_t q = t / n, c = t - q * n;
            t = q;
#pragma unroll
            for (int o = 0; o < NOPS; o++) off[o] += static_cast<size_t>(c) * strides[o][d];
        }
    } else {
        for (int d = rank - 1; d >= 0 && i != 0; d--) {
            const size_t q = i / dims[d], c = i - q * dims[d];
            i = q;
#pragma unroll
            for (int o = 0; o < NOPS; o++) off[o] += c * strides[o][d];
        }
    }
}

// ---- broadcast binary: info = [dims | a strides | b strides] ------------------------------------------------
template <typename X, typename Y, typename O, typename F>
__device__ __forceinline__ void binary_body(size_t n, size_t rank_, const size_t* info, const X* a, const Y* b, O* out, F f) {
    const int rank = static_cast<int>(rank_);
    const size_t* dims = info;
    const size_t* const strides[2] = {info + rank, info + 2 * rank};
    const bool small = n <= 0xffffffffull;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t off[2];
        offsets_of<2>(i, dims, strides, rank, small, off);
        out[i] = f(a[off[0]], b[off[1]]);
    }
}

// in-place b = f(alpha, a, beta, b): info = [dims | a strides | b strides]
template <typename T, typename F>
__device__ __forceinline__ void binary_inplace_body(T alpha, T beta, size_t n, size_t rank_, const size_t* info, const T* a, T* b, F f) {
    const int rank = static_cast<int>(rank_);
    const size_t* dims = info;
    const size_t* const strides[2] = {info + rank, info + 2 * rank};
    const bool small = n <= 0xffffffffull;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t off[2];
        offsets_of<2>(i, dims, strides, rank, small, off);
        b[off[1]] = f(alpha, a[off[0]], beta, b[off[1]]);
    }
}

// ---- broadcast ternary (Where): info = [dims | x | y | z strides] ----------------------------------------------
template <typename T, typename Z>
__device__ __forceinline__ void where_body(size_t n, size_t rank_, const size_t* info, const T* x, const T* y, const Z* z, T* out) {
    const int rank = static_cast<int>(rank_);
    const size_t* dims = info;
    const size_t* const strides[3] = {info + rank, info + 2 * rank, info + 3 * rank};
    const bool small = n <= 0xffffffffull;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t off[3];
        offsets_of<3>(i, dims, strides, rank, small, off);
        const T xv = x[off[0]];
        const T yv = y[off[1]];
        out[i] = z[off[2]] ? xv : yv;
    }
}

// ---- contiguous unary / cast ------------------------------------------------------------------------------------
template <typename I, typename O, typename F>
__device__ __forceinline__ void unary_body(size_t n, const I* in, O* out, F f) {
    for (size_t i = global_tid(); i < n; i += grid_threads()) out[i] = f(in[i]);
}

// static_cast between arithmetic types, through float for f16, `x != 0` into bool
template <typename O>
struct Cast {
    template <typename I>
    __device__ __forceinline__ O operator()(I x) const {
        if constexpr (std::is_same<O, bool>::value) {
            return x == I(0) ? false : true;
        } else {
            return static_cast<O>(x);
        }
    }
    __device__ __forceinline__ O operator()(__half x) const {
        if constexpr (std::is_same<O, bool>::value) {
            return __half2float(x) == 0.0f ? false : true;
        } else {
            return static_cast<O>(__half2float(x));
        }
    }
};
template <>
struct Cast<__half> {
    template <typename I>
    __device__ __forceinline__ __half operator()(I x) const { return __float2half(static_cast<float>(x)); }
};

// ---- Expand: info = [in shape | in strides | out shape | out strides], right-aligned broadcast ---------------
template <typename T>
__device__ __forceinline__ void expand_body(size_t n, size_t in_rank_, size_t out_rank_, const size_t* info, const T* in, T* out) {
    const int in_rank = static_cast<int>(in_rank_), out_rank = static_cast<int>(out_rank_);
    const size_t *ishape = info, *istr = info + in_rank, *oshape = info + 2 * in_rank, *ostr = info + 2 * in_rank + out_rank;
    const int lead = out_rank - in_rank;
    const bool small = n <= 0xffffffffull;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t src = 0, dst = 0;
        if (small) {  // 32-bit divides; stop once the remaining index is zero
            uint32_t t = static_cast<uint32_t>(i);
            for (int d = out_rank - 1; d >= 0 && t != 0; d--) {
                const uint32_t m = static_cast<uint32_t>(oshape[d]);
                const uint32_t q = t / m, c = t - q * m;
                t = q;
                dst += static_cast<size_t>(c) * ostr[d];
                const int id = d - lead;
                if (id >= 0 && ishape[id] != 1) src += static_cast<size_t>(c) * istr[id];
            }
        } else {
            size_t t = i;
            for (int d = out_rank - 1; d >= 0; d--) {
                const size_t q = t / oshape[d], c = t - q * oshape[d];
                t = q;
                dst += c * ostr[d];
                const int id = d - lead;
                if (id >= 0 && ishape[id] != 1) src += c * istr[id];
            }
        }
        out[dst] = in[src];
    }
}

// ---- Transpose: info = [dst dims | src strides | dst strides]; dst dim d walks src stride perm[d] ------------------
template <typename T>
__device__ __forceinline__ void transpose_body(size_t n, size_t rank_, const size_t* info, const size_t* perm, const T* src, T* dst) {
    const int rank = static_cast<int>(rank_);
    const size_t *dims = info, *sstr = info + rank, *dstr = info + 2 * rank;
    const bool small = n <= 0xffffffffull;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t so = 0, dof = 0;
        if (small) {  // 32-bit divides; stop once the remaining index is zero
            uint32_t t = static_cast<uint32_t>(i);
            for (int d = rank - 1; d >= 0 && t != 0; d--) {
                const uint32_t m = static_cast<uint32_t>(dims[d]);
                const uint32_t q = t / m, c = t - q * m;
                t = q;
                so += static_cast<size_t>(c) * sstr[perm[d]];
                dof += static_cast<size_t>(c) * dstr[d];
            }
        } else {
            size_t t = i;
            for (int d = rank - 1; d >= 0; d--) {
                const size_t q = t / dims[d], c = t - q * dims[d];
                t = q;
                so += c * sstr[perm[d]];
                dof += c * dstr[d];
            }
        }
        dst[dof] = src[so];
    }
}

// ---- Slice: info = [in shape | in strides | out shape | (unused)]; starts / ends / axes / steps are device arrays
// holding the op's raw inputs (negative values, INT_MIN / INT_MAX sentinels); axes / steps may be null.
template <typename T, typename I>
__device__ __forceinline__ void slice_body(size_t n, size_t axes_len, size_t rank_, const size_t* info, const T* in, const I* starts,
                                           const I* ends, const I* axes, const I* steps, T* out) {
    const int rank = static_cast<int>(rank_);
    if (global_tid() >= n || rank > 8) return;
    const size_t *ishape = info, *istr = info + rank, *oshape = info + 2 * rank;
    I first[8], last[8], step[8];
    for (int d = 0; d < rank; d++) {
        first[d] = 0;
        last[d] = static_cast<I>(ishape[d]);
        step[d] = 1;
    }
    const int given = static_cast<int>(axes_len ? axes_len : rank_);
    for (int k = 0; k < given; k++) {
        int ax = k;
        if (axes_len) ax = static_cast<int>(axes[k] < 0 ? axes[k] + rank : axes[k]);
        if (steps) step[ax] = steps[k];
        const I dim = static_cast<I>(ishape[ax]);
        const bool fwd = step[ax] >= 0;
        I s = starts[k];
        if (s < 0) s += dim;
        if (s < 0) s = 0;
        if (fwd && s > dim) s = dim;
        if (!fwd && s >= dim) s = dim - 1;
        first[ax] = s;
        I e = ends[k];
        if (e < 0) e += dim;
        if (e < -1) e = -1;
        if (fwd && e > dim) e = dim;
        if (!fwd && e >= dim) e = dim - 1;
        last[ax] = e;
    }
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t t = i, src = 0;
        bool inside = true;
        for (int d = rank - 1; d >= 0 && inside; d--) {
            const size_t q = t / oshape[d];
            const I pos = step[d] * static_cast<I>(t - q * oshape[d]) + first[d];
            t = q;
            inside = step[d] > 0 ? pos < last[d] : step[d] < 0 ? pos >= last[d] : true;
            src += static_cast<size_t>(pos) * istr[d];
        }
        if (inside) out[i] = in[src];
    }
}

// ---- Trilu on a [batch, rows, cols] view: info = [dims | strides] --------------------------------------------
template <typename T>
__device__ __forceinline__ void trilu_body(size_t n, bool upper, int64_t k, const size_t* info, const T* in, T* out) {
    const size_t *dims = info, *str = info + 3;
    for (size_t i = global_tid(); i < n; i += grid_threads()) {
        size_t t = i;
        const size_t col = t % dims[2];
        t /= dims[2];
        const size_t row = t % dims[1];
        const size_t b = t / dims[1];
        const size_t off = b * str[0] + row * str[1] + col * str[2];
        const int64_t diag = static_cast<int64_t>(col) - static_cast<int64_t>(row);
        const bool keep = upper ? diag >= k : diag <= k;
        out[off] = keep ? in[off] : T(0);
    }
}

// ---- ReduceMean, one thread per output: info = [shape | strides], axes = reduced dims -----------------------------
// LOAD converts an element to the accumulator type, STORE converts the (double) mean back.
template <typename T, typename ACC, typename LOAD, typename STORE>
__device__ __forceinline__ void reduce_mean_body(const size_t* axes, size_t num_axes, size_t rank_, const size_t* info, const T* in,
                                                 size_t reduced, size_t n_out, T* out, LOAD load, STORE store) {
    const int rank = static_cast<int>(rank_);
    if (rank > MAX_RANK) return;
    const size_t *shape = info, *str = info + rank;
    bool red[MAX_RANK];
    for (int d = 0; d < rank; d++) red[d] = false;
    for (size_t a = 0; a < num_axes; a++) red[axes[a]] = true;
    // reduced dims, innermost first, for the odometer
    int rdim[MAX_RANK], nr = 0;
    for (int d = rank - 1; d >= 0; d--)
        if (red[d] && shape[d] != 1) rdim[nr++] = d;
    for (size_t o = global_tid(); o < n_out; o += grid_threads()) {
        size_t t = o, base = 0;
        for (int d = rank - 1; d >= 0; d--)
            if (!red[d]) {
                const size_t q = t / shape[d];
                base += (t - q * shape[d]) * str[d];
                t = q;
            }
        ACC acc = 0;
        size_t cnt[MAX_RANK];
        for (int j = 0; j < nr; j++) cnt[j] = 0;
        size_t off = base;
        for (size_t e = 0; e < reduced; e++) {
            acc += load(in[off]);
            for (int j = 0; j < nr; j++) {  // advance the odometer over the reduced dims
                off += str[rdim[j]];
                if (++cnt[j] < shape[rdim[j]]) break;
                off -= cnt[j] * str[rdim[j]];
                cnt[j] = 0;
            }
        }
        out[o] = store(static_cast<double>(acc) / static_cast<double>(reduced));
    }
}

// ---- ScatterND, one thread per index tuple; info = [data shape | data strides | indices shape | indices strides |
// updates shape | updates strides]; *error: 1 = index out of range, 2 = slice past the end of data ---------------------
template <typename T, typename F>
__device__ __forceinline__ void scatter_nd_body(size_t n_tuples, size_t data_len, size_t data_rank, size_t idx_rank, size_t upd_rank,
                                                const size_t* info, const int64_t* indices, const T* updates, T* output, int* error, F f) {
    if (*error) return;
    const size_t *dshape = info, *dstr = info + data_rank;
    const size_t *ishape = info + 2 * data_rank, *istr = ishape + idx_rank;
    const size_t *ushape = info + 2 * data_rank + 2 * idx_rank, *ustr = ushape + upd_rank;
    const size_t tuple = idx_rank > 1 ? ishape[idx_rank - 1] : 1;
    const int prefix = static_cast<int>(idx_rank > 1 ? idx_rank - 1 : 1);
    size_t slice = 1;
    for (size_t d = prefix; d < upd_rank; d++) slice *= ushape[d];
    for (size_t tIdx = global_tid(); tIdx < n_tuples; tIdx += grid_threads()) {
        size_t t = tIdx, ioff = 0, uoff = 0;
        for (int d = prefix - 1; d >= 0; d--) {
            const size_t q = t / ishape[d];
            ioff += (t - q * ishape[d]) * istr[d];
            t = q;
        }
        t = tIdx;
        for (int d = prefix - 1; d >= 0; d--) {
            const size_t q = t / ushape[d];
            uoff += (t - q * ushape[d]) * ustr[d];
            t = q;
        }
        size_t doff = 0;
        for (size_t j = 0; j < tuple; j++) {
            int64_t ix = indices[ioff + j];
            const int64_t dim = static_cast<int64_t>(dshape[j]);
            if (ix < 0) ix += dim;
            if (ix < 0 || ix >= dim) {
                *error = 1;
                return;
            }
            doff += static_cast<size_t>(ix) * dstr[j];
        }
        if (doff + slice > data_len) {
            *error = 2;
            return;
        }
        for (size_t j = 0; j < slice; j++) output[doff + j] = f(updates[uoff + j], output[doff + j]);
    }
}

}  // namespace t1
