// ReduceMean and Softmax.
//
// ReduceMean (reference: one thread per output, serial double accumulation,
// cuda/src/ptx/headers/aggregation_op_macros.cuh:29-47) becomes a cooperative reduction: the dims
// are collapsed into alternating kept / reduced groups, and
//   - if the innermost group is reduced, a group of G threads (a warp, a quarter-CTA or a CTA)
//     owns one output, walks the reduction space with 128-bit loads and combines with
//     shfl.sync (+ one shared-memory hop across warps);
//   - if the innermost group is kept, consecutive threads own consecutive outputs so that every
//     load is coalesced, and each thread walks the reduction space serially.
// Accumulation stays in double (uint64 for the integer variants, which the reference computes as
// unsigned, cuda/src/ptx/reduce_mean.cu:8-9) and the order is fixed, so results are deterministic
// and within one rounding of the reference's sequential double sum.
//
// Softmax (reference: cudnnSoftmaxForward, cuda/src/kernels/softmax.rs:26-34) is a single pass for
// rows that fit the register budget of their thread group: one read of the row, max and sum by
// warp shuffles, one write.  Longer rows take an online max/sum pass and a second read (from L2).
#include "common.cuh"

namespace rmlk {

// ---------------------------------------------------------------------------------------------
// group reductions: G threads (a power of two, 32..1024, G <= blockDim.x) cooperate
// ---------------------------------------------------------------------------------------------
struct SumOp {
    template <typename T> __device__ static T op(T a, T b) { return a + b; }
};
struct MaxOp {
    template <typename T> __device__ static T op(T a, T b) { return a > b ? a : b; }
};

__device__ __forceinline__ double shfl_xor_t(double v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ __forceinline__ float shfl_xor_t(float v, int m) { return __shfl_xor_sync(0xffffffffu, v, m); }
__device__ __forceinline__ uint64_t shfl_xor_t(uint64_t v, int m) {
    return static_cast<uint64_t>(__shfl_xor_sync(0xffffffffu, static_cast<unsigned long long>(v), m));
}

template <typename Op, typename T>
__device__ __forceinline__ T warp_reduce(T v) {
#pragma unroll
    for (int m = 16; m >= 1; m >>= 1) v = Op::op(v, shfl_xor_t(v, m));
    return v;
}

// All G threads of the group get the result.  `smem` holds blockDim.x/32 slots of T.
template <typename Op, int G, typename T>
__device__ __forceinline__ T group_reduce(T v, T* smem, T identity) {
    v = warp_reduce<Op>(v);
    if constexpr (G > 32) {
        constexpr int WPG = G / 32;  // warps per group
        const int warp = threadIdx.x >> 5;
        const int lane = threadIdx.x & 31;
        const int gbase = (warp / WPG) * WPG;
        __syncthreads();
        if (lane == 0) smem[warp] = v;
        __syncthreads();
        T w = lane < WPG ? smem[gbase + lane] : identity;
        v = warp_reduce<Op>(w);
    }
    return v;
}

// ---------------------------------------------------------------------------------------------
// ReduceMean
// ---------------------------------------------------------------------------------------------
constexpr int RM_MAX_GROUPS = RMLK_MAX_RANK;

struct RmParams {
    int n_kept, n_red;                    // number of kept / reduced groups
    uint64_t kept_dim[RM_MAX_GROUPS];     // innermost first
    int64_t kept_stride[RM_MAX_GROUPS];
    uint64_t red_dim[RM_MAX_GROUPS];      // innermost first
    int64_t red_stride[RM_MAX_GROUPS];
    uint64_t n_out, n_red_total;
};

template <typename T> struct RmAcc { using type = double; };
template <> struct RmAcc<uint32_t> { using type = uint64_t; };
template <> struct RmAcc<uint64_t> { using type = uint64_t; };

template <typename T> __device__ __forceinline__ typename RmAcc<T>::type rm_in(T x) { return static_cast<typename RmAcc<T>::type>(x); }
template <> __device__ __forceinline__ double rm_in<__half>(__half x) { return static_cast<double>(__half2float(x)); }

template <typename T> __device__ __forceinline__ T rm_out(double div) { return static_cast<T>(div); }
template <> __device__ __forceinline__ __half rm_out<__half>(double div) { return __float2half(static_cast<float>(div)); }

__device__ __forceinline__ int64_t rm_offset(uint64_t idx, int n, const uint64_t* dim, const int64_t* stride) {
    int64_t off = 0;
    for (int j = 0; j < n; j++) {
        const uint64_t q = idx / dim[j];
        off += static_cast<int64_t>(idx - q * dim[j]) * stride[j];
        idx = q;
    }
    return off;
}

// Innermost group reduced and contiguous: G threads per output, V elements per load.
template <typename T, int G, int V, int BLOCK>
__global__ void __launch_bounds__(BLOCK) reduce_mean_row_kernel(RmParams p, const T* __restrict__ in, T* __restrict__ out) {
    dep_sync();
    using Acc = typename RmAcc<T>::type;
    __shared__ Acc smem[BLOCK / 32];
    constexpr int ROWS = BLOCK / G;
    const int g = threadIdx.x / G;
    const int t = threadIdx.x % G;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * ROWS + g;
    const bool live = row < p.n_out;
    Acc acc = 0;
    if (live) {
        const int64_t base = rm_offset(row, p.n_kept, p.kept_dim, p.kept_stride);
        const uint64_t inner = p.red_dim[0];
        const uint64_t outer = p.n_red_total / inner;
        for (uint64_t o = 0; o < outer; o++) {
            const int64_t ob = base + (p.n_red > 1 ? rm_offset(o, p.n_red - 1, p.red_dim + 1, p.red_stride + 1) : 0);
            const T* src = in + ob;
            for (uint64_t i = static_cast<uint64_t>(t) * V; i < inner; i += static_cast<uint64_t>(G) * V) {
                const Pack<T, V> v = load_pack<T, V>(src + i);
#pragma unroll
                for (int e = 0; e < V; e++) acc += rm_in<T>(v.v[e]);
            }
        }
    }
    acc = group_reduce<SumOp, G, Acc>(acc, smem, Acc(0));
    if (live && t == 0) {
        const double div = static_cast<double>(acc) / static_cast<double>(p.n_red_total);
        out[row] = rm_out<T>(div);
    }
}

// Innermost group kept: one thread per output, coalesced across threads, serial over the reduction.
template <typename T>
__global__ void __launch_bounds__(256) reduce_mean_col_kernel(RmParams p, const T* __restrict__ in, T* __restrict__ out) {
    dep_sync();
    using Acc = typename RmAcc<T>::type;
    const uint64_t o = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (o >= p.n_out) return;
    const int64_t base = rm_offset(o, p.n_kept, p.kept_dim, p.kept_stride);
    Acc acc = 0;
    if (p.n_red == 1) {
        const int64_t rs = p.red_stride[0];
        for (uint64_t r = 0; r < p.n_red_total; r++) acc += rm_in<T>(in[base + static_cast<int64_t>(r) * rs]);
    } else {
        for (uint64_t r = 0; r < p.n_red_total; r++) acc += rm_in<T>(in[base + rm_offset(r, p.n_red, p.red_dim, p.red_stride)]);
    }
    const double div = static_cast<double>(acc) / static_cast<double>(p.n_red_total);
    out[o] = rm_out<T>(div);
}

// Any layout, few outputs: G threads per output with strided (non-vector) loads.
template <typename T, int G, int BLOCK>
__global__ void __launch_bounds__(BLOCK) reduce_mean_generic_kernel(RmParams p, const T* __restrict__ in, T* __restrict__ out) {
    dep_sync();
    using Acc = typename RmAcc<T>::type;
    __shared__ Acc smem[BLOCK / 32];
    constexpr int ROWS = BLOCK / G;
    const int g = threadIdx.x / G;
    const int t = threadIdx.x % G;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * ROWS + g;
    const bool live = row < p.n_out;
    Acc acc = 0;
    if (live) {
        const int64_t base = rm_offset(row, p.n_kept, p.kept_dim, p.kept_stride);
        for (uint64_t r = t; r < p.n_red_total; r += G) acc += rm_in<T>(in[base + rm_offset(r, p.n_red, p.red_dim, p.red_stride)]);
    }
    acc = group_reduce<SumOp, G, Acc>(acc, smem, Acc(0));
    if (live && t == 0) {
        const double div = static_cast<double>(acc) / static_cast<double>(p.n_red_total);
        out[row] = rm_out<T>(div);
    }
}

template <typename T>
static int reduce_mean_typed(cudaStream_t st, int rank, const int64_t* shape, int num_axes, const int64_t* axes,
                             const T* in, T* out) {
    bool reduced[RMLK_MAX_RANK] = {false};
    for (int i = 0; i < num_axes; i++) {
        if (axes[i] < 0 || axes[i] >= rank) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: axis out of bounds");
        if (reduced[axes[i]]) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: duplicate axis");
        reduced[axes[i]] = true;
    }
    // dense strides, drop size-1 dims, merge neighbours of the same kind
    int64_t stride[RMLK_MAX_RANK];
    int64_t run = 1;
    for (int d = rank - 1; d >= 0; d--) {
        stride[d] = run;
        run *= shape[d];
    }
    struct Grp { uint64_t dim; int64_t stride; bool red; };
    Grp grp[RMLK_MAX_RANK];
    int ng = 0;
    for (int d = 0; d < rank; d++) {
        if (shape[d] == 1) continue;
        if (ng > 0 && grp[ng - 1].red == reduced[d]) {  // dense input: neighbouring dims always merge
            grp[ng - 1].dim *= static_cast<uint64_t>(shape[d]);
            grp[ng - 1].stride = stride[d];
        } else {
            grp[ng++] = {static_cast<uint64_t>(shape[d]), stride[d], reduced[d]};
        }
    }
    RmParams p;
    p.n_kept = p.n_red = 0;
    p.n_out = p.n_red_total = 1;
    for (int i = ng - 1; i >= 0; i--) {
        if (grp[i].red) {
            p.red_dim[p.n_red] = grp[i].dim;
            p.red_stride[p.n_red++] = grp[i].stride;
            p.n_red_total *= grp[i].dim;
        } else {
            p.kept_dim[p.n_kept] = grp[i].dim;
            p.kept_stride[p.n_kept++] = grp[i].stride;
            p.n_out *= grp[i].dim;
        }
    }
    if (run == 0) return RMLK_OK;  // empty input: nothing to write (output is empty or undefined)
    if (p.n_red == 0) {
        // Nothing (or only size-1 dims) reduced: mean of one element is the element itself.
        p.n_red = 1;
        p.red_dim[0] = 1;
        p.red_stride[0] = 1;
    }
    const bool inner_reduced = ng > 0 && grp[ng - 1].red;
    if (inner_reduced) {
        const uint64_t inner = p.red_dim[0];
        constexpr int V = 16 / sizeof(T);
        bool vec = (inner % V == 0) && aligned_to(in, 16);
        for (int j = 0; j < p.n_kept && vec; j++) vec = (p.kept_stride[j] % V == 0);
        for (int j = 1; j < p.n_red && vec; j++) vec = (p.red_stride[j] % V == 0);
        const uint64_t work = p.n_red_total;
        const bool many_rows = p.n_out >= static_cast<uint64_t>(sm_count()) * 64;
#define RM_LAUNCH(G, VV)                                                                              \
    do {                                                                                              \
        constexpr int ROWS = 256 / (G);                                                               \
        const unsigned grid = static_cast<unsigned>((p.n_out + ROWS - 1) / ROWS);                     \
        launch_dep(reduce_mean_row_kernel<T, G, VV, 256>, dim3(grid), dim3(256), 0, st, p, in, out);                      \
    } while (0)
        if (work <= 256 || (work <= 2048 && many_rows)) {
            if (vec) RM_LAUNCH(32, V); else RM_LAUNCH(32, 1);
        } else {
            if (vec) RM_LAUNCH(256, V); else RM_LAUNCH(256, 1);
        }
#undef RM_LAUNCH
        RMLK_CHECK_LAUNCH("reduce_mean_row_kernel");
        return RMLK_OK;
    }
    // innermost group kept
    if (p.n_out >= static_cast<uint64_t>(sm_count()) * 256 || p.n_red_total <= 32) {
        const unsigned grid = static_cast<unsigned>((p.n_out + 255) / 256);
        launch_dep(reduce_mean_col_kernel<T>, dim3(grid), dim3(256), 0, st, p, in, out);
        RMLK_CHECK_LAUNCH("reduce_mean_col_kernel");
    } else {
        constexpr int G = 32;
        const unsigned grid = static_cast<unsigned>((p.n_out + (256 / G) - 1) / (256 / G));
        launch_dep(reduce_mean_generic_kernel<T, G, 256>, dim3(grid), dim3(256), 0, st, p, in, out);
        RMLK_CHECK_LAUNCH("reduce_mean_generic_kernel");
    }
    return RMLK_OK;
}

// ---------------------------------------------------------------------------------------------
// Softmax
// ---------------------------------------------------------------------------------------------
__device__ __forceinline__ float sm_exp(float x) { return expf(x); }
__device__ __forceinline__ double sm_exp(double x) { return exp(x); }

// Register-resident single pass (f32): the row is held as NP packs of 4 per thread.
template <int G, int NP, int BLOCK>
__global__ void __launch_bounds__(BLOCK) softmax_f32_regs_kernel(uint64_t rows, uint32_t cols, const float* __restrict__ in,
                                                                float* __restrict__ out) {
    dep_sync();
    __shared__ float smem[BLOCK / 32];
    constexpr int ROWS = BLOCK / G;
    const int g = threadIdx.x / G;
    const int t = threadIdx.x % G;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * ROWS + g;
    const bool live = row < rows;
    const float* src = in + row * cols;
    float* dst = out + row * cols;
    Pack<float, 4> buf[NP];
    float mx = -INFINITY;
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const uint32_t c = (static_cast<uint32_t>(i) * G + t) * 4;
        if (live && c < cols) {
            buf[i] = load_pack<float, 4>(src + c);
#pragma unroll
            for (int e = 0; e < 4; e++) mx = fmaxf(mx, buf[i].v[e]);
        }
    }
    mx = group_reduce<MaxOp, G, float>(mx, smem, -INFINITY);
    float sum = 0.f;
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const uint32_t c = (static_cast<uint32_t>(i) * G + t) * 4;
        if (live && c < cols) {
#pragma unroll
            for (int e = 0; e < 4; e++) {
                buf[i].v[e] = expf(buf[i].v[e] - mx);
                sum += buf[i].v[e];
            }
        }
    }
    sum = group_reduce<SumOp, G, float>(sum, smem, 0.f);
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const uint32_t c = (static_cast<uint32_t>(i) * G + t) * 4;
        if (live && c < cols) {
#pragma unroll
            for (int e = 0; e < 4; e++) buf[i].v[e] = buf[i].v[e] / sum;
            store_pack<float, 4>(dst + c, buf[i]);
        }
    }
}

// Any dtype / width: online (max, sum) pass, then a second read.  C is the compute type.
template <typename T, typename C, int G, int BLOCK>
__global__ void __launch_bounds__(BLOCK) softmax_generic_kernel(uint64_t rows, uint64_t cols, const T* __restrict__ in,
                                                               T* __restrict__ out) {
    dep_sync();
    __shared__ C smem[BLOCK / 32];
    constexpr int ROWS = BLOCK / G;
    const int g = threadIdx.x / G;
    const int t = threadIdx.x % G;
    const uint64_t row = static_cast<uint64_t>(blockIdx.x) * ROWS + g;
    const bool live = row < rows;
    const T* src = in + row * cols;
    T* dst = out + row * cols;
    C mx = -INFINITY;
    if (live)
        for (uint64_t c = t; c < cols; c += G) {
            const C v = static_cast<C>(src[c]);
            mx = v > mx ? v : mx;
        }
    mx = group_reduce<MaxOp, G, C>(mx, smem, static_cast<C>(-INFINITY));
    C sum = 0;
    if (live)
        for (uint64_t c = t; c < cols; c += G) sum += sm_exp(static_cast<C>(src[c]) - mx);
    sum = group_reduce<SumOp, G, C>(sum, smem, C(0));
    if (live)
        for (uint64_t c = t; c < cols; c += G) dst[c] = static_cast<T>(sm_exp(static_cast<C>(src[c]) - mx) / sum);
}

// Softmax over the middle dim of [outer, C, inner]: one thread per (outer, inner) position, coalesced
// along `inner`, three passes over C (the column stays in L1/L2).
__global__ void __launch_bounds__(256) softmax_strided_kernel(uint64_t outer, uint64_t C, uint64_t inner, const float* __restrict__ in,
                                                              float* __restrict__ out) {
    dep_sync();
    const uint64_t i = static_cast<uint64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= outer * inner) return;
    const uint64_t o = i / inner, r = i - o * inner;
    const float* src = in + o * C * inner + r;
    float* dst = out + o * C * inner + r;
    float mx = -INFINITY;
    for (uint64_t c = 0; c < C; c++) mx = fmaxf(mx, src[c * inner]);
    float sum = 0.f;
    for (uint64_t c = 0; c < C; c++) sum += expf(src[c * inner] - mx);
    for (uint64_t c = 0; c < C; c++) dst[c * inner] = expf(src[c * inner] - mx) / sum;
}

template <int G, int NP>
static void softmax_regs_launch(cudaStream_t st, uint64_t rows, uint32_t cols, const float* in, float* out) {
    constexpr int ROWS = 256 / G;
    const unsigned grid = static_cast<unsigned>((rows + ROWS - 1) / ROWS);
    launch_dep(softmax_f32_regs_kernel<G, NP, 256>, dim3(grid), dim3(256), 0, st, rows, cols, in, out);
}

}  // namespace rmlk

using namespace rmlk;

extern "C" int rmlk_b200_reduce_mean(rmlk_stream_t stream, int dtype, int rank, const int64_t* shape, int num_axes,
                                     const int64_t* axes, const void* in, void* out) {
    if (rank < 1 || rank > RMLK_MAX_RANK || !shape) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: rank must be in [1, 8]");
    if (num_axes < 0 || num_axes > rank || (num_axes > 0 && !axes)) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: bad axes");
    for (int i = 0; i < rank; i++)
        if (shape[i] < 0) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: negative dimension");
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "reduce_mean: NULL tensor pointer");
    cudaStream_t st = as_stream(stream);
    switch (dtype) {
        case RMLK_F16: return reduce_mean_typed<__half>(st, rank, shape, num_axes, axes, static_cast<const __half*>(in), static_cast<__half*>(out));
        case RMLK_F32: return reduce_mean_typed<float>(st, rank, shape, num_axes, axes, static_cast<const float*>(in), static_cast<float*>(out));
        case RMLK_F64: return reduce_mean_typed<double>(st, rank, shape, num_axes, axes, static_cast<const double*>(in), static_cast<double*>(out));
        case RMLK_I32: case RMLK_U32:
            return reduce_mean_typed<uint32_t>(st, rank, shape, num_axes, axes, static_cast<const uint32_t*>(in), static_cast<uint32_t*>(out));
        case RMLK_I64: case RMLK_U64:
            return reduce_mean_typed<uint64_t>(st, rank, shape, num_axes, axes, static_cast<const uint64_t*>(in), static_cast<uint64_t*>(out));
        default: return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for reduce_mean");
    }
}

extern "C" int rmlk_b200_softmax(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* in, void* out) {
    if (rows < 0 || cols < 0) return fail(RMLK_ERR_INVALID_ARG, "softmax: negative extent");
    if (rows == 0 || cols == 0) return RMLK_OK;
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "softmax: NULL tensor pointer");
    cudaStream_t st = as_stream(stream);
    const uint64_t R = static_cast<uint64_t>(rows), C = static_cast<uint64_t>(cols);
    if (dtype == RMLK_F32) {
        const float* src = static_cast<const float*>(in);
        float* dst = static_cast<float*>(out);
        const bool vec = (C % 4 == 0) && aligned_to(in, 16) && aligned_to(out, 16) && C <= 8192;
        if (vec) {
            const uint32_t c32 = static_cast<uint32_t>(C);
            if (C <= 128) softmax_regs_launch<32, 1>(st, R, c32, src, dst);
            else if (C <= 256) softmax_regs_launch<32, 2>(st, R, c32, src, dst);
            else if (C <= 512) softmax_regs_launch<32, 4>(st, R, c32, src, dst);
            else if (C <= 1024) softmax_regs_launch<32, 8>(st, R, c32, src, dst);
            else if (C <= 2048) softmax_regs_launch<256, 2>(st, R, c32, src, dst);
            else if (C <= 4096) softmax_regs_launch<256, 4>(st, R, c32, src, dst);
            else softmax_regs_launch<256, 8>(st, R, c32, src, dst);
            RMLK_CHECK_LAUNCH("softmax_f32_regs_kernel");
            return RMLK_OK;
        }
        if (C <= 1024) {
            launch_dep(softmax_generic_kernel<float, float, 32, 256>, dim3(static_cast<unsigned>((R + 7) / 8)), dim3(256), 0, st, R, C, src, dst);
        } else {
            launch_dep(softmax_generic_kernel<float, float, 256, 256>, dim3(static_cast<unsigned>(R)), dim3(256), 0, st, R, C, src, dst);
        }
        RMLK_CHECK_LAUNCH("softmax_generic_kernel<float>");
        return RMLK_OK;
    }
    if (dtype == RMLK_F16) {
        launch_dep(softmax_generic_kernel<__half, float, 256, 256>, dim3(static_cast<unsigned>(R)), dim3(256), 0, st, 
            R, C, static_cast<const __half*>(in), static_cast<__half*>(out));
        RMLK_CHECK_LAUNCH("softmax_generic_kernel<half>");
        return RMLK_OK;
    }
    if (dtype == RMLK_F64) {
        launch_dep(softmax_generic_kernel<double, double, 256, 256>, dim3(static_cast<unsigned>(R)), dim3(256), 0, st, 
            R, C, static_cast<const double*>(in), static_cast<double*>(out));
        RMLK_CHECK_LAUNCH("softmax_generic_kernel<double>");
        return RMLK_OK;
    }
    return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for softmax");
}

extern "C" int rmlk_b200_softmax_strided(rmlk_stream_t stream, int dtype, int64_t outer, int64_t channels, int64_t inner,
                                         const void* in, void* out) {
    if (outer < 0 || channels < 0 || inner < 0) return fail(RMLK_ERR_INVALID_ARG, "softmax: negative extent");
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for softmax");
    if (outer == 0 || channels == 0 || inner == 0) return RMLK_OK;
    if (!in || !out) return fail(RMLK_ERR_INVALID_ARG, "softmax: NULL tensor pointer");
    if (inner == 1) return rmlk_b200_softmax(stream, dtype, outer, channels, in, out);
    const uint64_t n = static_cast<uint64_t>(outer) * inner;
    launch_dep(softmax_strided_kernel, dim3(static_cast<unsigned>((n + 255) / 256)), dim3(256), 0, as_stream(stream), 
        static_cast<uint64_t>(outer), static_cast<uint64_t>(channels), static_cast<uint64_t>(inner), static_cast<const float*>(in),
        static_cast<float*>(out));
    RMLK_CHECK_LAUNCH("softmax_strided_kernel");
    return RMLK_OK;
}
