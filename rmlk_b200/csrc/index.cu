// Indexing / layout kernels: Gather, ScatterND, Slice, Transpose, Concat, Trilu, Range, Fill.
//
// All of them move bytes; none does arithmetic on the payload except ScatterND's reductions.  The
// copy kernels therefore work on "units" of 16 / 8 / 4 / 2 / 1 bytes — the widest that divides
// every contiguous run and pointer offset involved — so that a KV-cache append or an embedding
// gather moves 128 bits per thread regardless of the element type.
//
// Slice and the Transposes that keep the innermost dimension are strided-read / dense-write copies
// and run on the broadcast elementwise engine (elementwise.cuh) with the identity functor; its
// stride-collapse turns e.g. perm (0,2,1,3) on [B,S,H,D] into rows of D contiguous elements.
// Transposes that move the innermost dimension go through a padded shared-memory tile so that both
// the global reads and the global writes are coalesced.
#include "elementwise.cuh"

namespace rmlk {

struct CopyF { template <typename T> __device__ static T apply(T x) { return x; } };

static int strided_copy(cudaStream_t st, int elem_size, int rank, const int64_t* out_shape, const int64_t* in_strides,
                        const void* in, void* out) {
    switch (elem_size) {
        case 1: return ew_launch1<CopyF, uint8_t, uint8_t>(st, rank, out_shape, in_strides, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out));
        case 2: return ew_launch1<CopyF, uint16_t, uint16_t>(st, rank, out_shape, in_strides, static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out));
        case 4: return ew_launch1<CopyF, uint32_t, uint32_t>(st, rank, out_shape, in_strides, static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out));
        case 8: return ew_launch1<CopyF, uint64_t, uint64_t>(st, rank, out_shape, in_strides, static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out));
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "element size must be 1, 2, 4 or 8");
    }
}

// Widest unit (bytes) dividing all the given byte counts / addresses.
static int pick_unit(std::initializer_list<uint64_t> vals) {
    int u = 16;
    for (uint64_t v : vals)
        while (u > 1 && (v % static_cast<uint64_t>(u)) != 0) u >>= 1;
    return u;
}

// ---------------------------------------------------------------------------------------------
// Gather
// ---------------------------------------------------------------------------------------------
template <typename U, typename I>
__global__ void __launch_bounds__(256) gather_kernel(uint64_t total_units, uint32_t row_units, FastDiv row_div, uint32_t n_idx,
                                                     FastDiv idx_div, int64_t axis_dim, uint64_t in_outer_units,
                                                     const U* __restrict__ data, const I* __restrict__ indices,
                                                     U* __restrict__ out, int* __restrict__ status) {
    dep_sync();
    const uint64_t u = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (u >= total_units) return;
    uint32_t row, c, o, j;
    row_div.divmod(static_cast<uint32_t>(u), row, c);   // row = o * n_idx + j
    idx_div.divmod(row, o, j);
    int64_t ix = static_cast<int64_t>(indices[j]);
    if (ix < 0) ix += axis_dim;
    if (ix < 0 || ix >= axis_dim) {
        if (status && c == 0) *status = 1;
        return;
    }
    out[u] = data[static_cast<uint64_t>(o) * in_outer_units + static_cast<uint64_t>(ix) * row_units + c];
}

// Rows of a multiple of four units: a thread takes four consecutive units of one row - one index load, then four data
// loads in flight (with one unit per thread the two dependent loads of every thread left a gather of 8 KB rows at 0.80 of
// the copy bandwidth).
template <typename U, typename I>
__global__ void __launch_bounds__(256) gather4_kernel(uint64_t total_quads, uint32_t row_quads, FastDiv row_div, uint32_t n_idx,
                                                      FastDiv idx_div, int64_t axis_dim, uint64_t in_outer_units,
                                                      const U* __restrict__ data, const I* __restrict__ indices,
                                                      U* __restrict__ out, int* __restrict__ status) {
    dep_sync();
    const uint64_t q = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (q >= total_quads) return;
    uint32_t row, c, o, j;
    row_div.divmod(static_cast<uint32_t>(q), row, c);   // row = o * n_idx + j; c = quad inside the row
    idx_div.divmod(row, o, j);
    int64_t ix = static_cast<int64_t>(indices[j]);
    if (ix < 0) ix += axis_dim;
    if (ix < 0 || ix >= axis_dim) {
        if (status && c == 0) *status = 1;
        return;
    }
    const U* __restrict__ src = data + static_cast<uint64_t>(o) * in_outer_units + (static_cast<uint64_t>(ix) * row_quads + c) * 4;
    const U v0 = src[0], v1 = src[1], v2 = src[2], v3 = src[3];
    U* __restrict__ dst = out + q * 4;
    dst[0] = v0; dst[1] = v1; dst[2] = v2; dst[3] = v3;
}

template <typename U>
static int gather_units(cudaStream_t st, int idx_dtype, uint64_t total, uint32_t row_units, uint32_t n_idx, int64_t axis_dim,
                        const void* data, const void* indices, void* out, int* status) {
    const uint64_t in_outer = static_cast<uint64_t>(axis_dim) * row_units;
    if (row_units % 4 == 0 && row_units >= 16 && total / 4 < (1ull << 32)) {
        const uint64_t quads = total / 4;
        const uint32_t row_quads = row_units / 4;
        const unsigned grid4 = static_cast<unsigned>((quads + 255) / 256);
        if (idx_dtype == RMLK_I64)
            launch_dep(gather4_kernel<U, int64_t>, dim3(grid4), dim3(256), 0, st, quads, row_quads, FastDiv(row_quads), n_idx, FastDiv(n_idx), axis_dim,
                       in_outer, static_cast<const U*>(data), static_cast<const int64_t*>(indices), static_cast<U*>(out), status);
        else
            launch_dep(gather4_kernel<U, int32_t>, dim3(grid4), dim3(256), 0, st, quads, row_quads, FastDiv(row_quads), n_idx, FastDiv(n_idx), axis_dim,
                       in_outer, static_cast<const U*>(data), static_cast<const int32_t*>(indices), static_cast<U*>(out), status);
        RMLK_CHECK_LAUNCH("gather4_kernel");
        return RMLK_OK;
    }
    const unsigned grid = static_cast<unsigned>((total + 255) / 256);
    if (idx_dtype == RMLK_I64)
        launch_dep(gather_kernel<U, int64_t>, dim3(grid), dim3(256), 0, st, total, row_units, FastDiv(row_units), n_idx, FastDiv(n_idx), axis_dim, in_outer,
                                                        static_cast<const U*>(data), static_cast<const int64_t*>(indices), static_cast<U*>(out), status);
    else
        launch_dep(gather_kernel<U, int32_t>, dim3(grid), dim3(256), 0, st, total, row_units, FastDiv(row_units), n_idx, FastDiv(n_idx), axis_dim, in_outer,
                                                        static_cast<const U*>(data), static_cast<const int32_t*>(indices), static_cast<U*>(out), status);
    RMLK_CHECK_LAUNCH("gather_kernel");
    return RMLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Concat: up to CONCAT_MAX inputs per launch, table passed by value
// ---------------------------------------------------------------------------------------------
constexpr int CONCAT_MAX = 16;
struct ConcatTable {
    const void* src[CONCAT_MAX];
    uint64_t row_units[CONCAT_MAX];   // units per outer row of this input
    uint64_t dst_off[CONCAT_MAX];     // unit offset of this input inside an output row
    FastDiv row_div[CONCAT_MAX];      // by row_units, used when every index fits 31 bits
    uint64_t out_row_units;
    uint64_t outer;
    int narrow;
};

template <typename U>
__global__ void __launch_bounds__(256) concat_kernel(ConcatTable t, U* __restrict__ out) {
    dep_sync();
    const int i = blockIdx.y;
    const uint64_t ru = t.row_units[i];
    const uint64_t total = ru * t.outer;
    const U* __restrict__ src = static_cast<const U*>(t.src[i]);
    for (uint64_t u = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; u < total; u += static_cast<uint64_t>(gridDim.x) * 256) {
        uint64_t o, c;
        if (t.narrow) {
            uint32_t q, r;
            t.row_div[i].divmod(static_cast<uint32_t>(u), q, r);
            o = q;
            c = r;
        } else {
            o = u / ru;
            c = u - o * ru;
        }
        out[o * t.out_row_units + t.dst_off[i] + c] = src[u];
    }
}

// ---------------------------------------------------------------------------------------------
// Transpose through a shared-memory tile.  View: in[b][y][m][x] -> out[b'][x][m'][y] generalised as
//   in  offset = batch_in  + y * in_stride_y  + x            (x: input-innermost, stride 1)
//   out offset = batch_out + x * out_stride_x + y            (y: output-innermost, stride 1)
// with the remaining dims enumerated by blockIdx.z via a small (dim, in_stride, out_stride) table.
// ---------------------------------------------------------------------------------------------
struct TileParams {
    uint32_t nx, ny;
    int64_t in_stride_y, out_stride_x;
    int n_batch;
    uint64_t batch_dim[RMLK_MAX_RANK];
    int64_t batch_in[RMLK_MAX_RANK], batch_out[RMLK_MAX_RANK];
    uint64_t n_batches;
};

template <typename U>
__global__ void __launch_bounds__(256) transpose_tile_kernel(TileParams p, const U* __restrict__ in, U* __restrict__ out) {
    dep_sync();
    __shared__ U tile[32][33];
    const uint32_t tiles_x = (p.nx + 31) / 32;
    const uint32_t tiles_y = (p.ny + 31) / 32;
    const uint64_t tiles_per_batch = static_cast<uint64_t>(tiles_x) * tiles_y;
    const uint64_t total = tiles_per_batch * p.n_batches;
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;  // 32 x 8
    for (uint64_t tIdx = blockIdx.x; tIdx < total; tIdx += gridDim.x) {
        uint64_t b = tIdx / tiles_per_batch;
        const uint64_t r = tIdx - b * tiles_per_batch;
        const uint32_t by = static_cast<uint32_t>(r / tiles_x), bx = static_cast<uint32_t>(r - static_cast<uint64_t>(by) * tiles_x);
        int64_t in_b = 0, out_b = 0;
        for (int j = 0; j < p.n_batch; j++) {
            const uint64_t q = b / p.batch_dim[j];
            const uint64_t c = b - q * p.batch_dim[j];
            in_b += static_cast<int64_t>(c) * p.batch_in[j];
            out_b += static_cast<int64_t>(c) * p.batch_out[j];
            b = q;
        }
        const uint32_t x0 = bx * 32, y0 = by * 32;
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t y = y0 + ty + k * 8, x = x0 + tx;
            if (y < p.ny && x < p.nx) tile[ty + k * 8][tx] = in[in_b + static_cast<int64_t>(y) * p.in_stride_y + x];
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const uint32_t x = x0 + ty + k * 8, y = y0 + tx;
            if (y < p.ny && x < p.nx) out[out_b + static_cast<int64_t>(x) * p.out_stride_x + y] = tile[tx][ty + k * 8];
        }
        __syncthreads();
    }
}

// 4-byte elements through a 64 x 64 tile held as T[x][y] (pitch 64 words).  Word (x, y) lives at column
//   4 * ((y >> 2) ^ ((x >> 2) & 7)) + ((y ^ x) & 3)
// of row x: the 16-byte y-quads are XOR-swizzled with the x-quad index and the words inside a quad with the
// low bits of x.  With that placement all four access patterns are free of bank conflicts: 16-byte global
// loads scattered as scalar stores (8 x-quads x 4 rows per warp), scalar global loads (one row of 32 x per
// warp), 16-byte shared loads feeding 16-byte global stores (16 y-quads x 2 x per warp) and scalar loads
// (one x, 32 y per warp).  VIN / VOUT select 16-byte accesses on the input / output side; each needs that
// side's extent, stride and batch strides to be multiples of 4 and its base pointer 16-byte aligned (the
// host checks).  A side that fails the test, e.g. rows of odd length, uses coalesced 4-byte accesses.
__device__ __forceinline__ uint32_t tile64_col(uint32_t x, uint32_t y) { return 4 * ((y >> 2) ^ ((x >> 2) & 7)) + ((y ^ x) & 3); }

template <bool VIN, bool VOUT>
__global__ void __launch_bounds__(256) transpose_tile64_kernel(TileParams p, const uint32_t* __restrict__ in, uint32_t* __restrict__ out) {
    dep_sync();
    __shared__ __align__(16) uint32_t tile[64 * 64];
    const uint32_t tiles_x = (p.nx + 63) / 64;
    const uint32_t tiles_y = (p.ny + 63) / 64;
    const uint64_t tiles_per_batch = static_cast<uint64_t>(tiles_x) * tiles_y;
    const uint64_t total = tiles_per_batch * p.n_batches;
    const uint32_t lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (uint64_t tIdx = blockIdx.x; tIdx < total; tIdx += gridDim.x) {
        uint64_t b = tIdx / tiles_per_batch;
        const uint64_t r = tIdx - b * tiles_per_batch;
        const uint32_t by = static_cast<uint32_t>(r / tiles_x), bx = static_cast<uint32_t>(r - static_cast<uint64_t>(by) * tiles_x);
        int64_t in_b = 0, out_b = 0;
        for (int j = 0; j < p.n_batch; j++) {
            const uint64_t q = b / p.batch_dim[j];
            const uint64_t c = b - q * p.batch_dim[j];
            in_b += static_cast<int64_t>(c) * p.batch_in[j];
            out_b += static_cast<int64_t>(c) * p.batch_out[j];
            b = q;
        }
        const uint32_t x0 = bx * 64, y0 = by * 64;
        if constexpr (VIN) {
            uint4 v[4];
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t u = warp + 8 * i;
                const uint32_t xl = 4 * (8 * (u & 1) + (lane & 7)), yl = 4 * (u >> 1) + (lane >> 3);
                v[i] = make_uint4(0, 0, 0, 0);
                if (x0 + xl < p.nx && y0 + yl < p.ny)
                    v[i] = ld_stream_u4(reinterpret_cast<const uint4*>(in + in_b + static_cast<int64_t>(y0 + yl) * p.in_stride_y + x0 + xl));
            }
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t u = warp + 8 * i;
                const uint32_t xl = 4 * (8 * (u & 1) + (lane & 7)), yl = 4 * (u >> 1) + (lane >> 3);
                tile[(xl + 0) * 64 + tile64_col(xl + 0, yl)] = v[i].x;
                tile[(xl + 1) * 64 + tile64_col(xl + 1, yl)] = v[i].y;
                tile[(xl + 2) * 64 + tile64_col(xl + 2, yl)] = v[i].z;
                tile[(xl + 3) * 64 + tile64_col(xl + 3, yl)] = v[i].w;
            }
        } else {
            uint32_t v[16];
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t yl = warp + 8 * i;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t xl = lane + 32 * h;
                    v[2 * i + h] = 0;
                    if (x0 + xl < p.nx && y0 + yl < p.ny) v[2 * i + h] = __ldg(in + in_b + static_cast<int64_t>(y0 + yl) * p.in_stride_y + x0 + xl);
                }
            }
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t yl = warp + 8 * i;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t xl = lane + 32 * h;
                    tile[xl * 64 + tile64_col(xl, yl)] = v[2 * i + h];
                }
            }
        }
        __syncthreads();
        if constexpr (VOUT) {
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const uint32_t xl = 2 * (warp + 8 * i) + (lane >> 4), yq = lane & 15;
                if (x0 + xl < p.nx && y0 + 4 * yq < p.ny) {
                    uint4 w = *reinterpret_cast<const uint4*>(&tile[xl * 64 + 4 * (yq ^ ((xl >> 2) & 7))]);
                    // undo the in-quad permutation: slot e holds y = 4 * yq + (e ^ (x & 3))
                    if (xl & 1) { uint32_t t = w.x; w.x = w.y; w.y = t; t = w.z; w.z = w.w; w.w = t; }
                    if (xl & 2) { uint32_t t = w.x; w.x = w.z; w.z = t; t = w.y; w.y = w.w; w.w = t; }
                    *reinterpret_cast<uint4*>(out + out_b + static_cast<int64_t>(x0 + xl) * p.out_stride_x + y0 + 4 * yq) = w;
                }
            }
        } else {
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const uint32_t xl = warp + 8 * i;
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const uint32_t yl = lane + 32 * h;
                    if (x0 + xl < p.nx && y0 + yl < p.ny)
                        out[out_b + static_cast<int64_t>(x0 + xl) * p.out_stride_x + y0 + yl] = tile[xl * 64 + tile64_col(xl, yl)];
                }
            }
        }
        __syncthreads();
    }
}

// ---------------------------------------------------------------------------------------------
// Trilu
// ---------------------------------------------------------------------------------------------
template <typename T, int V>
__global__ void __launch_bounds__(256) trilu_kernel(uint64_t total_packs, uint32_t col_packs, FastDiv col_div, uint32_t rows,
                                                    FastDiv row_div, int upper, int64_t k, const T* __restrict__ in,
                                                    T* __restrict__ out) {
    dep_sync();
    const uint64_t u = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (u >= total_packs) return;
    uint32_t rowlin, cp, b, r;
    col_div.divmod(static_cast<uint32_t>(u), rowlin, cp);
    row_div.divmod(rowlin, b, r);
    (void)b;
    const int64_t c0 = static_cast<int64_t>(cp) * V;
    const int64_t edge = static_cast<int64_t>(r) + k;  // upper keeps c >= edge, lower keeps c <= edge
    Pack<T, V> v;
    const bool any = upper ? (c0 + V - 1 >= edge) : (c0 <= edge);
    if (any) {
        v = load_pack<T, V>(in + u * V);
#pragma unroll
        for (int e = 0; e < V; e++) {
            const int64_t c = c0 + e;
            const bool keep = upper ? (c >= edge) : (c <= edge);
            if (!keep) v.v[e] = T(0);
        }
    } else {
#pragma unroll
        for (int e = 0; e < V; e++) v.v[e] = T(0);
    }
    store_pack<T, V>(out + u * V, v);
}

template <typename T>
static int trilu_typed(cudaStream_t st, int64_t batch, int64_t rows, int64_t cols, int upper, int64_t k, const void* in, void* out) {
    constexpr int VMAX = 16 / sizeof(T);
    const uint64_t n = static_cast<uint64_t>(batch) * rows * cols;
    const bool vec = (cols % VMAX == 0) && aligned_to(in, 16) && aligned_to(out, 16);
    const uint64_t packs = vec ? n / VMAX : n;
    if (packs > EW_NARROW_LIMIT) return fail(RMLK_ERR_INVALID_ARG, "trilu: tensor too large");
    const unsigned grid = static_cast<unsigned>((packs + 255) / 256);
    if (vec)
        launch_dep(trilu_kernel<T, VMAX>, dim3(grid), dim3(256), 0, st, packs, static_cast<uint32_t>(cols / VMAX), FastDiv(static_cast<uint32_t>(cols / VMAX)),
                                                    static_cast<uint32_t>(rows), FastDiv(static_cast<uint32_t>(rows)), upper, k,
                                                    static_cast<const T*>(in), static_cast<T*>(out));
    else
        launch_dep(trilu_kernel<T, 1>, dim3(grid), dim3(256), 0, st, packs, static_cast<uint32_t>(cols), FastDiv(static_cast<uint32_t>(cols)),
                                                 static_cast<uint32_t>(rows), FastDiv(static_cast<uint32_t>(rows)), upper, k,
                                                 static_cast<const T*>(in), static_cast<T*>(out));
    RMLK_CHECK_LAUNCH("trilu_kernel");
    return RMLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Range / Fill
// ---------------------------------------------------------------------------------------------
template <typename T> struct RangeOp {
    __device__ static T at(T start, T delta, uint64_t i) { return start + static_cast<T>(i) * delta; }
};
// Floating types: the host loop the reference runs (backend/range.rs:195-205) rounds the product
// and then the sum; keep the two roundings (no FMA contraction).
template <> struct RangeOp<float> {
    __device__ static float at(float start, float delta, uint64_t i) { return __fadd_rn(start, __fmul_rn(static_cast<float>(i), delta)); }
};
template <> struct RangeOp<double> {
    __device__ static double at(double start, double delta, uint64_t i) { return __dadd_rn(start, __dmul_rn(static_cast<double>(i), delta)); }
};
template <> struct RangeOp<__half> {
    __device__ static __half at(__half start, __half delta, uint64_t i) {
        return __hadd(start, __hmul(__float2half(static_cast<float>(i)), delta));
    }
};

template <typename T>
__global__ void __launch_bounds__(256) range_kernel(uint64_t n, T start, T delta, T* __restrict__ out) {
    dep_sync();
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * 256)
        out[i] = RangeOp<T>::at(start, delta, i);
}

template <typename U>
__global__ void __launch_bounds__(256) fill_kernel(uint64_t n, U value, U* __restrict__ out) {
    dep_sync();
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < n; i += static_cast<uint64_t>(gridDim.x) * 256) out[i] = value;
}

struct SmallWords { uint64_t w[32]; };
__global__ void store_small_kernel(SmallWords v, int n, uint64_t* __restrict__ out) {
    dep_sync();
    if (threadIdx.x < n) out[threadIdx.x] = v.w[threadIdx.x];
}

// ---------------------------------------------------------------------------------------------
// ScatterND
// ---------------------------------------------------------------------------------------------
struct ScatterParams {
    int k;
    int64_t dim[RMLK_MAX_RANK];
    int64_t stride[RMLK_MAX_RANK];  // element strides of data for the first k dims
    uint64_t slice_len;
    uint64_t total;                 // n_tuples * slice_len
};

template <int RED, typename T>
__device__ __forceinline__ T scatter_apply(T in, T outv) {
    if constexpr (RED == RMLK_SCATTER_NONE) return in;
    else if constexpr (RED == RMLK_SCATTER_ADD) return in + outv;
    else if constexpr (RED == RMLK_SCATTER_MUL) return in * outv;
    else if constexpr (RED == RMLK_SCATTER_MAX) return in > outv ? in : outv;
    else return in < outv ? in : outv;
}

template <int RED, typename T>
__global__ void __launch_bounds__(256) scatter_nd_kernel(ScatterParams p, const int64_t* __restrict__ indices,
                                                         const T* __restrict__ updates, T* __restrict__ out, int* __restrict__ status) {
    dep_sync();
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= p.total) return;
    const uint64_t t = i / p.slice_len;
    const uint64_t e = i - t * p.slice_len;
    int64_t off = 0;
    for (int j = 0; j < p.k; j++) {
        int64_t ix = indices[t * p.k + j];
        if (ix < 0) ix += p.dim[j];
        if (ix < 0 || ix >= p.dim[j]) {
            if (status && e == 0) *status = 1;
            return;
        }
        off += ix * p.stride[j];
    }
    const T in = updates[i];
    if constexpr (RED == RMLK_SCATTER_NONE) {
        out[off + e] = in;
    } else {
        out[off + e] = scatter_apply<RED, T>(in, out[off + e]);
    }
}

// Plain assignment of whole slices in 16-byte units (slice length, bases and every slice offset multiples of 16 bytes):
// four times fewer, four times wider accesses than the element kernel.
__global__ void __launch_bounds__(256) scatter_nd_units_kernel(ScatterParams p, uint32_t unit_elems, const int64_t* __restrict__ indices,
                                                               const uint4* __restrict__ updates, uint4* __restrict__ out, int* __restrict__ status) {
    dep_sync();
    const uint64_t slice_units = p.slice_len / unit_elems;
    const uint64_t total = p.total / unit_elems;
    for (uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<uint64_t>(gridDim.x) * 256) {
        const uint64_t t = i / slice_units;
        const uint64_t e = i - t * slice_units;
        int64_t off = 0;
        bool ok = true;
        for (int j = 0; j < p.k; j++) {
            int64_t ix = indices[t * p.k + j];
            if (ix < 0) ix += p.dim[j];
            if (ix < 0 || ix >= p.dim[j]) {
                if (status && e == 0) *status = 1;
                ok = false;
                break;
            }
            off += ix * p.stride[j];
        }
        if (ok) out[static_cast<uint64_t>(off) / unit_elems + e] = updates[i];
    }
}

template <typename T>
static int scatter_typed(cudaStream_t st, int reduction, const ScatterParams& p, const void* indices, const void* updates, void* out, int* status) {
    const unsigned grid = static_cast<unsigned>((p.total + 255) / 256);
    const int64_t* ix = static_cast<const int64_t*>(indices);
    const T* up = static_cast<const T*>(updates);
    T* o = static_cast<T*>(out);
    switch (reduction) {
        case RMLK_SCATTER_NONE: launch_dep(scatter_nd_kernel<RMLK_SCATTER_NONE, T>, dim3(grid), dim3(256), 0, st, p, ix, up, o, status); break;
        case RMLK_SCATTER_ADD: launch_dep(scatter_nd_kernel<RMLK_SCATTER_ADD, T>, dim3(grid), dim3(256), 0, st, p, ix, up, o, status); break;
        case RMLK_SCATTER_MUL: launch_dep(scatter_nd_kernel<RMLK_SCATTER_MUL, T>, dim3(grid), dim3(256), 0, st, p, ix, up, o, status); break;
        case RMLK_SCATTER_MAX: launch_dep(scatter_nd_kernel<RMLK_SCATTER_MAX, T>, dim3(grid), dim3(256), 0, st, p, ix, up, o, status); break;
        case RMLK_SCATTER_MIN: launch_dep(scatter_nd_kernel<RMLK_SCATTER_MIN, T>, dim3(grid), dim3(256), 0, st, p, ix, up, o, status); break;
        default: return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: unknown reduction");
    }
    RMLK_CHECK_LAUNCH("scatter_nd_kernel");
    return RMLK_OK;
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_gather(rmlk_stream_t stream, int elem_size, int idx_dtype, int64_t outer, int64_t axis_dim,
                                int64_t inner, int64_t n_idx, const void* data, const void* indices, void* out, int* status) {
    if (outer < 0 || axis_dim < 0 || inner < 0 || n_idx < 0) return fail(RMLK_ERR_INVALID_ARG, "gather: negative extent");
    if (idx_dtype != RMLK_I32 && idx_dtype != RMLK_I64) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for gather indices");
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "gather: element size must be 1, 2, 4 or 8");
    if (outer == 0 || inner == 0 || n_idx == 0) return RMLK_OK;
    if (!data || !indices || !out) return fail(RMLK_ERR_INVALID_ARG, "gather: NULL tensor pointer");
    const uint64_t row_bytes = static_cast<uint64_t>(inner) * elem_size;
    const int unit = pick_unit({row_bytes, reinterpret_cast<uintptr_t>(data), reinterpret_cast<uintptr_t>(out)});
    const uint64_t row_units = row_bytes / unit;
    const uint64_t total = static_cast<uint64_t>(outer) * n_idx * row_units;
    if (total > EW_NARROW_LIMIT || row_units > EW_NARROW_LIMIT) return fail(RMLK_ERR_INVALID_ARG, "gather: output too large");
    cudaStream_t st = as_stream(stream);
    const uint32_t ru = static_cast<uint32_t>(row_units), ni = static_cast<uint32_t>(n_idx);
    switch (unit) {
        case 16: return gather_units<uint4>(st, idx_dtype, total, ru, ni, axis_dim, data, indices, out, status);
        case 8: return gather_units<uint64_t>(st, idx_dtype, total, ru, ni, axis_dim, data, indices, out, status);
        case 4: return gather_units<uint32_t>(st, idx_dtype, total, ru, ni, axis_dim, data, indices, out, status);
        case 2: return gather_units<uint16_t>(st, idx_dtype, total, ru, ni, axis_dim, data, indices, out, status);
        default: return gather_units<uint8_t>(st, idx_dtype, total, ru, ni, axis_dim, data, indices, out, status);
    }
}

extern "C" int rmlk_b200_concat(rmlk_stream_t stream, int elem_size, int n_inputs, int64_t outer, int64_t inner,
                                const int64_t* axis_dims, const void* const* inputs, void* out) {
    if (n_inputs < 1 || !axis_dims || !inputs) return fail(RMLK_ERR_INVALID_ARG, "concat: needs at least one input");
    if (outer < 0 || inner < 0) return fail(RMLK_ERR_INVALID_ARG, "concat: negative extent");
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "concat: element size must be 1, 2, 4 or 8");
    uint64_t total_axis = 0;
    for (int i = 0; i < n_inputs; i++) {
        if (axis_dims[i] < 0) return fail(RMLK_ERR_INVALID_ARG, "concat: negative axis extent");
        total_axis += static_cast<uint64_t>(axis_dims[i]);
    }
    if (outer == 0 || inner == 0 || total_axis == 0) return RMLK_OK;
    if (!out) return fail(RMLK_ERR_INVALID_ARG, "concat: NULL output");
    // unit: widest that divides every row length, every row offset and every base address
    int unit = 16;
    {
        uint64_t off = 0;
        auto shrink = [&](uint64_t v) { while (unit > 1 && v % static_cast<uint64_t>(unit)) unit >>= 1; };
        shrink(reinterpret_cast<uintptr_t>(out));
        shrink(total_axis * inner * elem_size);
        for (int i = 0; i < n_inputs; i++) {
            if (axis_dims[i] == 0) continue;
            if (!inputs[i]) return fail(RMLK_ERR_INVALID_ARG, "concat: NULL input");
            shrink(reinterpret_cast<uintptr_t>(inputs[i]));
            shrink(static_cast<uint64_t>(axis_dims[i]) * inner * elem_size);
            shrink(off * inner * elem_size);
            off += static_cast<uint64_t>(axis_dims[i]);
        }
    }
    cudaStream_t st = as_stream(stream);
    uint64_t off_elems = 0;
    int i = 0;
    while (i < n_inputs) {
        ConcatTable t;
        int cnt = 0;
        uint64_t max_units = 0;
        t.out_row_units = total_axis * inner * elem_size / unit;
        t.outer = static_cast<uint64_t>(outer);
        for (; i < n_inputs && cnt < CONCAT_MAX; i++) {
            const uint64_t ax = static_cast<uint64_t>(axis_dims[i]);
            if (ax == 0) continue;
            t.src[cnt] = inputs[i];
            t.row_units[cnt] = ax * inner * elem_size / unit;
            t.dst_off[cnt] = off_elems * inner * elem_size / unit;
            t.row_div[cnt] = FastDiv(static_cast<uint32_t>(t.row_units[cnt] <= EW_NARROW_LIMIT ? t.row_units[cnt] : 1));
            if (t.row_units[cnt] * t.outer > max_units) max_units = t.row_units[cnt] * t.outer;
            off_elems += ax;
            cnt++;
        }
        if (cnt == 0) break;
        t.narrow = max_units <= EW_NARROW_LIMIT ? 1 : 0;
        dim3 grid(flat_grid(static_cast<int64_t>(max_units), 256, 16), cnt);
        switch (unit) {
            case 16: launch_dep(concat_kernel<uint4>, dim3(grid), dim3(256), 0, st, t, static_cast<uint4*>(out)); break;
            case 8: launch_dep(concat_kernel<uint64_t>, dim3(grid), dim3(256), 0, st, t, static_cast<uint64_t*>(out)); break;
            case 4: launch_dep(concat_kernel<uint32_t>, dim3(grid), dim3(256), 0, st, t, static_cast<uint32_t*>(out)); break;
            case 2: launch_dep(concat_kernel<uint16_t>, dim3(grid), dim3(256), 0, st, t, static_cast<uint16_t*>(out)); break;
            default: launch_dep(concat_kernel<uint8_t>, dim3(grid), dim3(256), 0, st, t, static_cast<uint8_t*>(out)); break;
        }
        RMLK_CHECK_LAUNCH("concat_kernel");
    }
    return RMLK_OK;
}

extern "C" int rmlk_b200_slice_params(int rank, const int64_t* in_shape, int n, const int64_t* starts, const int64_t* ends,
                                      const int64_t* axes, const int64_t* steps, int64_t* out_starts, int64_t* out_steps,
                                      int64_t* out_shape) {
    if (rank < 1 || rank > RMLK_MAX_RANK || !in_shape || !out_starts || !out_steps || !out_shape)
        return fail(RMLK_ERR_INVALID_ARG, "slice: rank must be in [1, 8]");
    if (n < 0 || n > rank || (n > 0 && (!starts || !ends))) return fail(RMLK_ERR_INVALID_ARG, "slice: bad starts/ends");
    for (int d = 0; d < rank; d++) {
        out_starts[d] = 0;
        out_steps[d] = 1;
        out_shape[d] = in_shape[d];
    }
    for (int kx = 0; kx < n; kx++) {
        int64_t axis = axes ? axes[kx] : kx;
        if (axis < 0) axis += rank;
        if (axis < 0 || axis >= rank) return fail(RMLK_ERR_INVALID_ARG, "slice: axis out of range");
        const int64_t step = steps ? steps[kx] : 1;
        if (step == 0) return fail(RMLK_ERR_INVALID_ARG, "slice: zero step");
        const int64_t dim = in_shape[axis];
        int64_t start = starts[kx];
        if (start < 0) start += dim;
        if (start < 0) start = 0;
        if (step > 0 && start > dim) start = dim;
        else if (step < 0 && start >= dim) start = dim - 1;
        int64_t end = ends[kx];
        if (end < 0) end += dim;
        if (end < -1) end = -1;
        if (step > 0 && end > dim) end = dim;
        else if (step < 0 && end >= dim) end = dim - 1;
        int64_t cnt;
        if ((step < 0 && start < end) || (step > 0 && start >= end)) cnt = 0;
        else if (step > 0) cnt = (end - start + step - 1) / step;
        else cnt = (start - end + (-step) - 1) / (-step);
        out_starts[axis] = start;
        out_steps[axis] = step;
        out_shape[axis] = cnt;
    }
    return RMLK_OK;
}

extern "C" int rmlk_b200_slice(rmlk_stream_t stream, int elem_size, int rank, const int64_t* in_shape, const int64_t* out_shape,
                               const int64_t* starts, const int64_t* steps, const void* in, void* out) {
    if (rank < 1 || rank > RMLK_MAX_RANK || !in_shape || !out_shape || !starts || !steps)
        return fail(RMLK_ERR_INVALID_ARG, "slice: rank must be in [1, 8]");
    for (int d = 0; d < rank; d++)
        if (out_shape[d] == 0) return RMLK_OK;  // empty result: nothing to write
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "slice: NULL tensor pointer");
    int64_t in_stride[RMLK_MAX_RANK], eff[RMLK_MAX_RANK];
    int64_t run = 1, base = 0, n_out = 1;
    for (int d = rank - 1; d >= 0; d--) {
        in_stride[d] = run;
        run *= in_shape[d];
    }
    for (int d = 0; d < rank; d++) {
        if (out_shape[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "slice: negative output extent");
        n_out *= out_shape[d];
        if (out_shape[d] > 0) {
            const int64_t last = starts[d] + steps[d] * (out_shape[d] - 1);
            if (starts[d] < 0 || starts[d] >= in_shape[d] || last < 0 || last >= in_shape[d])
                return fail(RMLK_ERR_INVALID_ARG, "slice: range outside the input");
        }
        base += starts[d] * in_stride[d];
        eff[d] = steps[d] * in_stride[d];
    }
    if (n_out == 0) return RMLK_OK;
    const char* src = static_cast<const char*>(in) + base * elem_size;
    return strided_copy(as_stream(stream), elem_size, rank, out_shape, eff, src, out);
}

static int view_copy(cudaStream_t st, int elem_size, int n, int64_t* oshape, int64_t* ostr_in, const void* in, void* out);

// Dense copy of an arbitrary strided view: strides in elements, 0 = broadcast, negative allowed as long as
// every addressed element lies inside the caller's buffer.  Used by the host runtime to materialise a chain
// of Expand / Reshape / Transpose that was kept as a view (one copy instead of one per op).  The reference has
// no views: each of those ops copies (backend/expand.rs:49-216, backend/transpose.rs:44-178).
extern "C" int rmlk_b200_strided_copy(rmlk_stream_t stream, int elem_size, int rank, const int64_t* shape, const int64_t* strides,
                                      const void* in, void* out) {
    if (rank < 0 || rank > RMLK_MAX_RANK || (rank > 0 && (!shape || !strides))) return fail(RMLK_ERR_INVALID_ARG, "strided_copy: rank must be in [0, 8]");
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "strided_copy: element size must be 1, 2, 4 or 8");
    int64_t oshape[RMLK_MAX_RANK], ostr_in[RMLK_MAX_RANK];
    int n = 0;
    for (int d = 0; d < rank; d++) {
        if (shape[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "strided_copy: negative extent");
        if (shape[d] == 0) return RMLK_OK;
    }
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "strided_copy: NULL tensor pointer");
    for (int d = 0; d < rank; d++) {
        if (shape[d] == 1) continue;
        if (n > 0 && ostr_in[n - 1] == strides[d] * shape[d]) {
            oshape[n - 1] *= shape[d];
            ostr_in[n - 1] = strides[d];
        } else {
            oshape[n] = shape[d];
            ostr_in[n++] = strides[d];
        }
    }
    return view_copy(as_stream(stream), elem_size, n, oshape, ostr_in, in, out);
}

// Strided view -> strided view, one launch: element i (row-major over `shape`) is read at sum idx_d * in_strides[d]
// and written at sum idx_d * out_strides[d].  The host runtime uses it to put rows that exist only as a view (a
// block of columns of a wider MatMul result, permuted) straight into their slot of a carried cache, where the
// reference copies twice (backend/transpose.rs:44-178, then backend/concat.rs:28-198 over the whole cache).
struct Copy2Params {
    int rank;
    FastDiv div[RMLK_MAX_RANK];
    int64_t is[RMLK_MAX_RANK], os[RMLK_MAX_RANK];
};

template <typename U>
__global__ void __launch_bounds__(256) strided_copy2_kernel(Copy2Params p, uint32_t total, const U* __restrict__ in, U* __restrict__ out) {
    dep_sync();
    for (uint32_t i = blockIdx.x * 256u + threadIdx.x; i < total; i += gridDim.x * 256u) {
        uint32_t t = i;
        int64_t io = 0, oo = 0;
        for (int d = p.rank - 1; d >= 0; d--) {
            uint32_t q, r;
            p.div[d].divmod(t, q, r);
            t = q;
            io += static_cast<int64_t>(r) * p.is[d];
            oo += static_cast<int64_t>(r) * p.os[d];
        }
        out[oo] = in[io];
    }
}

extern "C" int rmlk_b200_strided_copy_to(rmlk_stream_t stream, int elem_size, int rank, const int64_t* shape, const int64_t* in_strides,
                                         const int64_t* out_strides, const void* in, void* out) {
    if (rank < 0 || rank > RMLK_MAX_RANK || (rank > 0 && (!shape || !in_strides || !out_strides)))
        return fail(RMLK_ERR_INVALID_ARG, "strided_copy_to: rank must be in [0, 8]");
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "strided_copy_to: element size must be 1, 2, 4 or 8");
    for (int d = 0; d < rank; d++) {
        if (shape[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "strided_copy_to: negative extent");
        if (shape[d] == 0) return RMLK_OK;
    }
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "strided_copy_to: NULL tensor pointer");
    // drop dims of size 1, merge neighbours that are contiguous on both sides
    int64_t dim[RMLK_MAX_RANK], is[RMLK_MAX_RANK], os[RMLK_MAX_RANK];
    int n = 0;
    for (int d = 0; d < rank; d++) {
        if (shape[d] == 1) continue;
        if (n > 0 && is[n - 1] == in_strides[d] * shape[d] && os[n - 1] == out_strides[d] * shape[d]) {
            dim[n - 1] *= shape[d];
            is[n - 1] = in_strides[d];
            os[n - 1] = out_strides[d];
        } else {
            dim[n] = shape[d];
            is[n] = in_strides[d];
            os[n++] = out_strides[d];
        }
    }
    if (n == 0) {
        dim[0] = 1; is[0] = 1; os[0] = 1;
        n = 1;
    }
    // 16-byte units when both sides walk the innermost dim contiguously and everything else keeps the alignment
    int unit = elem_size;
    if (is[n - 1] == 1 && os[n - 1] == 1) {
        for (int v = 16 / elem_size; v > 1; v /= 2) {
            bool ok = dim[n - 1] % v == 0 && reinterpret_cast<uintptr_t>(in) % (v * elem_size) == 0 && reinterpret_cast<uintptr_t>(out) % (v * elem_size) == 0;
            for (int d = 0; d + 1 < n && ok; d++) ok = is[d] % v == 0 && os[d] % v == 0;
            if (ok) {
                dim[n - 1] /= v;
                for (int d = 0; d + 1 < n; d++) {
                    is[d] /= v;
                    os[d] /= v;
                }
                unit = v * elem_size;
                break;
            }
        }
    }
    int64_t total = 1;
    Copy2Params p;
    p.rank = n;
    for (int d = 0; d < n; d++) {
        if (dim[d] > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "strided_copy_to: more than 2^31 units");
        total *= dim[d];
        if (total > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "strided_copy_to: more than 2^31 units");
        p.div[d] = FastDiv(static_cast<uint32_t>(dim[d]));
        p.is[d] = is[d];
        p.os[d] = os[d];
    }
    cudaStream_t st = as_stream(stream);
    const unsigned grid = flat_grid(total, 256, 16);
    const uint32_t tot = static_cast<uint32_t>(total);
    switch (unit) {
        case 1: launch_dep(strided_copy2_kernel<uint8_t>, dim3(grid), dim3(256), 0, st, p, tot, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out)); break;
        case 2: launch_dep(strided_copy2_kernel<uint16_t>, dim3(grid), dim3(256), 0, st, p, tot, static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out)); break;
        case 4: launch_dep(strided_copy2_kernel<uint32_t>, dim3(grid), dim3(256), 0, st, p, tot, static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out)); break;
        case 8: launch_dep(strided_copy2_kernel<uint64_t>, dim3(grid), dim3(256), 0, st, p, tot, static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out)); break;
        default: launch_dep(strided_copy2_kernel<uint4>, dim3(grid), dim3(256), 0, st, p, tot, static_cast<const uint4*>(in), static_cast<uint4*>(out)); break;
    }
    RMLK_CHECK_LAUNCH("strided_copy2_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_transpose(rmlk_stream_t stream, int elem_size, int rank, const int64_t* in_shape, const int64_t* perm,
                                   const void* in, void* out) {
    if (rank < 1 || rank > RMLK_MAX_RANK || !in_shape || !perm) return fail(RMLK_ERR_INVALID_ARG, "transpose: rank must be in [1, 8]");
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "transpose: NULL tensor pointer");
    if (elem_size != 1 && elem_size != 2 && elem_size != 4 && elem_size != 8) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "transpose: element size must be 1, 2, 4 or 8");
    bool seen[RMLK_MAX_RANK] = {false};
    int64_t in_stride[RMLK_MAX_RANK];
    int64_t run = 1;
    for (int d = rank - 1; d >= 0; d--) {
        in_stride[d] = run;
        run *= in_shape[d];
    }
    for (int d = 0; d < rank; d++) {
        if (perm[d] < 0 || perm[d] >= rank || seen[perm[d]]) return fail(RMLK_ERR_INVALID_ARG, "transpose: perm is not a permutation");
        seen[perm[d]] = true;
    }
    if (run == 0) return RMLK_OK;
    // output dims with the input stride each one walks; drop size-1 dims; merge runs
    int64_t oshape[RMLK_MAX_RANK], ostr_in[RMLK_MAX_RANK];
    int n = 0;
    for (int d = 0; d < rank; d++) {
        const int64_t sz = in_shape[perm[d]], s = in_stride[perm[d]];
        if (sz == 1) continue;
        if (n > 0 && ostr_in[n - 1] == s * sz) {
            oshape[n - 1] *= sz;
            ostr_in[n - 1] = s;
        } else {
            oshape[n] = sz;
            ostr_in[n++] = s;
        }
    }
    return view_copy(as_stream(stream), elem_size, n, oshape, ostr_in, in, out);
}

// out (dense, row-major over oshape[0..n)) = the view of `in` whose dim d walks ostr_in[d] elements (0 for a
// broadcast dim).  A view whose innermost stride is 1 goes to the strided-copy engine; one whose unit-stride
// dim sits elsewhere goes through a shared-memory tile so that both sides stay coalesced.
static int view_copy(cudaStream_t st, int elem_size, int n, int64_t* oshape, int64_t* ostr_in, const void* in, void* out) {
    if (n == 0) {
        oshape[0] = 1;
        ostr_in[0] = 1;
        n = 1;
    }
    int64_t run = 1;
    if (ostr_in[n - 1] == 1 || n == 1) return strided_copy(st, elem_size, n, oshape, ostr_in, in, out);
    // innermost dimension moves: find the output position whose input stride is 1
    int px = -1;
    for (int d = 0; d < n; d++)
        if (ostr_in[d] == 1) px = d;
    if (px < 0) return strided_copy(st, elem_size, n, oshape, ostr_in, in, out);  // cannot happen for a dense input
    int64_t out_stride[RMLK_MAX_RANK];
    run = 1;
    for (int d = n - 1; d >= 0; d--) {
        out_stride[d] = run;
        run *= oshape[d];
    }
    TileParams p;
    p.nx = static_cast<uint32_t>(oshape[px]);
    p.ny = static_cast<uint32_t>(oshape[n - 1]);
    if (oshape[px] > 0xffffffffll || oshape[n - 1] > 0xffffffffll) return strided_copy(st, elem_size, n, oshape, ostr_in, in, out);
    p.in_stride_y = ostr_in[n - 1];
    p.out_stride_x = out_stride[px];
    p.n_batch = 0;
    p.n_batches = 1;
    for (int d = n - 2; d >= 0; d--) {
        if (d == px) continue;
        p.batch_dim[p.n_batch] = static_cast<uint64_t>(oshape[d]);
        p.batch_in[p.n_batch] = ostr_in[d];
        p.batch_out[p.n_batch] = out_stride[d];
        p.n_batches *= static_cast<uint64_t>(oshape[d]);
        p.n_batch++;
    }
    if (elem_size == 4) {
        bool vin = p.nx % 4 == 0 && p.in_stride_y % 4 == 0 && reinterpret_cast<uintptr_t>(in) % 16 == 0;
        bool vout = p.ny % 4 == 0 && p.out_stride_x % 4 == 0 && reinterpret_cast<uintptr_t>(out) % 16 == 0;
        for (int j = 0; j < p.n_batch; j++) {
            vin = vin && p.batch_in[j] % 4 == 0;
            vout = vout && p.batch_out[j] % 4 == 0;
        }
        const uint64_t tiles64 = static_cast<uint64_t>((p.nx + 63) / 64) * ((p.ny + 63) / 64) * p.n_batches;
        const unsigned grid64 = static_cast<unsigned>(tiles64 < (1u << 30) ? tiles64 : (1u << 30));
        const uint32_t* src = static_cast<const uint32_t*>(in);
        uint32_t* dst = static_cast<uint32_t*>(out);
        if (vin && vout) launch_dep(transpose_tile64_kernel<true, true>, dim3(grid64), dim3(256), 0, st, p, src, dst);
        else if (vin) launch_dep(transpose_tile64_kernel<true, false>, dim3(grid64), dim3(256), 0, st, p, src, dst);
        else if (vout) launch_dep(transpose_tile64_kernel<false, true>, dim3(grid64), dim3(256), 0, st, p, src, dst);
        else launch_dep(transpose_tile64_kernel<false, false>, dim3(grid64), dim3(256), 0, st, p, src, dst);
        RMLK_CHECK_LAUNCH("transpose_tile64_kernel");
        return RMLK_OK;
    }
    const uint64_t tiles = static_cast<uint64_t>((p.nx + 31) / 32) * ((p.ny + 31) / 32) * p.n_batches;
    const unsigned grid = static_cast<unsigned>(tiles < (1u << 30) ? tiles : (1u << 30));
    switch (elem_size) {
        case 1: launch_dep(transpose_tile_kernel<uint8_t>, dim3(grid), dim3(256), 0, st, p, static_cast<const uint8_t*>(in), static_cast<uint8_t*>(out)); break;
        case 2: launch_dep(transpose_tile_kernel<uint16_t>, dim3(grid), dim3(256), 0, st, p, static_cast<const uint16_t*>(in), static_cast<uint16_t*>(out)); break;
        case 4: launch_dep(transpose_tile_kernel<uint32_t>, dim3(grid), dim3(256), 0, st, p, static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out)); break;
        default: launch_dep(transpose_tile_kernel<uint64_t>, dim3(grid), dim3(256), 0, st, p, static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out)); break;
    }
    RMLK_CHECK_LAUNCH("transpose_tile_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_trilu(rmlk_stream_t stream, int elem_size, int64_t batch, int64_t rows, int64_t cols, int upper,
                               int64_t k, const void* in, void* out) {
    if (batch < 0 || rows < 0 || cols < 0) return fail(RMLK_ERR_INVALID_ARG, "trilu: negative extent");
    if (batch == 0 || rows == 0 || cols == 0) return RMLK_OK;
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "trilu: NULL tensor pointer");
    if (rows > 0x7fffffffll || cols > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "trilu: matrix too large");
    cudaStream_t st = as_stream(stream);
    switch (elem_size) {
        case 1: return trilu_typed<uint8_t>(st, batch, rows, cols, upper, k, in, out);
        case 2: return trilu_typed<uint16_t>(st, batch, rows, cols, upper, k, in, out);
        case 4: return trilu_typed<uint32_t>(st, batch, rows, cols, upper, k, in, out);
        case 8: return trilu_typed<uint64_t>(st, batch, rows, cols, upper, k, in, out);
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "trilu: element size must be 1, 2, 4 or 8");
    }
}

extern "C" int rmlk_b200_range(rmlk_stream_t stream, int dtype, int64_t n, const void* start, const void* delta, void* out) {
    if (n < 0) return fail(RMLK_ERR_INVALID_ARG, "range: negative count");
    if (n == 0) return RMLK_OK;
    if (!start || !delta || !out) return fail(RMLK_ERR_INVALID_ARG, "range: NULL pointer");
    cudaStream_t st = as_stream(stream);
    const unsigned grid = flat_grid(n, 256, 32);  // grid-stride: a few thousand CTAs whatever n
#define RMLK_CASE(DT, T)                                                                                                   \
    case DT:                                                                                                               \
        launch_dep(range_kernel<T>, dim3(grid), dim3(256), 0, st, static_cast<uint64_t>(n), *static_cast<const T*>(start), *static_cast<const T*>(delta), static_cast<T*>(out)); \
        break;
    switch (dtype) {
        RMLK_CASE(RMLK_F16, __half)
        RMLK_CASE(RMLK_F32, float)
        RMLK_CASE(RMLK_F64, double)
        RMLK_CASE(RMLK_I32, int32_t)
        RMLK_CASE(RMLK_I64, int64_t)
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for range");
    }
#undef RMLK_CASE
    RMLK_CHECK_LAUNCH("range_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_fill(rmlk_stream_t stream, int elem_size, int64_t n, const void* value, void* out) {
    if (n < 0) return fail(RMLK_ERR_INVALID_ARG, "fill: negative count");
    if (n == 0) return RMLK_OK;
    if (!value || !out) return fail(RMLK_ERR_INVALID_ARG, "fill: NULL pointer");
    cudaStream_t st = as_stream(stream);
    const unsigned grid = flat_grid(n, 256, 16);
    switch (elem_size) {
        case 1: { uint8_t v; memcpy(&v, value, 1); launch_dep(fill_kernel<uint8_t>, dim3(grid), dim3(256), 0, st, static_cast<uint64_t>(n), v, static_cast<uint8_t*>(out)); break; }
        case 2: { uint16_t v; memcpy(&v, value, 2); launch_dep(fill_kernel<uint16_t>, dim3(grid), dim3(256), 0, st, static_cast<uint64_t>(n), v, static_cast<uint16_t*>(out)); break; }
        case 4: { uint32_t v; memcpy(&v, value, 4); launch_dep(fill_kernel<uint32_t>, dim3(grid), dim3(256), 0, st, static_cast<uint64_t>(n), v, static_cast<uint32_t*>(out)); break; }
        case 8: { uint64_t v; memcpy(&v, value, 8); launch_dep(fill_kernel<uint64_t>, dim3(grid), dim3(256), 0, st, static_cast<uint64_t>(n), v, static_cast<uint64_t*>(out)); break; }
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "fill: element size must be 1, 2, 4 or 8");
    }
    RMLK_CHECK_LAUNCH("fill_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_scatter_nd(rmlk_stream_t stream, int reduction, int dtype, int data_rank, const int64_t* data_shape,
                                    int64_t n_tuples, int k, const void* data, const void* indices, const void* updates,
                                    void* out, int* status) {
    if (data_rank < 1 || data_rank > RMLK_MAX_RANK || !data_shape) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: rank must be in [1, 8]");
    if (k < 1 || k > data_rank) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: index tuple longer than the data rank");
    if (n_tuples < 0) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: negative tuple count");
    if (!data || !out) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: NULL tensor pointer");
    const size_t es = dtype_size(dtype);
    cudaStream_t st = as_stream(stream);
    ScatterParams p;
    p.k = k;
    int64_t stride[RMLK_MAX_RANK];
    int64_t run = 1;
    for (int d = data_rank - 1; d >= 0; d--) {
        if (data_shape[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: negative dimension");
        stride[d] = run;
        run *= data_shape[d];
    }
    p.slice_len = 1;
    for (int d = k; d < data_rank; d++) p.slice_len *= static_cast<uint64_t>(data_shape[d]);
    for (int d = 0; d < k; d++) {
        p.dim[d] = data_shape[d];
        p.stride[d] = stride[d];
    }
    p.total = static_cast<uint64_t>(n_tuples) * p.slice_len;
    switch (dtype) {
        case RMLK_F16: case RMLK_F32: case RMLK_F64: case RMLK_I32: case RMLK_I64: break;
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for scatter_nd");
    }
    if (data != out && run > 0) RMLK_CUDA(cudaMemcpyAsync(out, data, static_cast<size_t>(run) * es, cudaMemcpyDeviceToDevice, st));
    if (p.total == 0 || run == 0) return RMLK_OK;
    if (!indices || !updates) return fail(RMLK_ERR_INVALID_ARG, "scatter_nd: NULL tensor pointer");
    if (reduction == RMLK_SCATTER_NONE && (p.slice_len * es) % 16 == 0 && aligned_to(out, 16) && aligned_to(updates, 16)) {
        // every slice then starts on a 16-byte boundary: the strides of the indexed dimensions are multiples of the slice length
        const uint32_t unit_elems = static_cast<uint32_t>(16 / es);
        const uint64_t units = p.total / unit_elems;
        launch_dep(scatter_nd_units_kernel, dim3(flat_grid(static_cast<int64_t>(units), 256, 16)), dim3(256), 0, st, p, unit_elems,
                   static_cast<const int64_t*>(indices), static_cast<const uint4*>(updates), static_cast<uint4*>(out), status);
        RMLK_CHECK_LAUNCH("scatter_nd_units_kernel");
        return RMLK_OK;
    }
    switch (dtype) {
        case RMLK_F16: return scatter_typed<__half>(st, reduction, p, indices, updates, out, status);
        case RMLK_F32: return scatter_typed<float>(st, reduction, p, indices, updates, out, status);
        case RMLK_F64: return scatter_typed<double>(st, reduction, p, indices, updates, out, status);
        case RMLK_I32: return scatter_typed<int32_t>(st, reduction, p, indices, updates, out, status);
        default: return scatter_typed<int64_t>(st, reduction, p, indices, updates, out, status);
    }
}

extern "C" int rmlk_b200_store_small(rmlk_stream_t stream, int n_words, const uint64_t* words, void* out) {
    if (n_words < 0 || n_words > 32) return fail(RMLK_ERR_INVALID_ARG, "store_small: at most 32 words");
    if (n_words == 0) return RMLK_OK;
    if (!words || !out || !aligned_to(out, 8)) return fail(RMLK_ERR_INVALID_ARG, "store_small: bad pointer");
    SmallWords v;
    for (int i = 0; i < 32; i++) v.w[i] = i < n_words ? words[i] : 0;
    launch_dep(store_small_kernel, dim3(1), dim3(32), 0, as_stream(stream), v, n_words, static_cast<uint64_t*>(out));
    RMLK_CHECK_LAUNCH("store_small_kernel");
    return RMLK_OK;
}
