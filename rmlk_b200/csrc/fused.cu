// Fused forms of op chains that an exported decoder graph spells out op by op.  Each kernel evaluates the same
// fp32 expressions, in the same order, as the chain of single-op kernels it stands for (same libm calls, no
// FMA contraction across op boundaries), so results agree with the op-by-op path to the last bit except for
// the summation order inside the row reductions.  The host runtime substitutes them when it recognises the
// chain (runtime/ops.cpp); the single-op entry points stay the reference-facing interface.
//
//   rmsnorm             Pow(x, 2) -> ReduceMean(last axis, keepdims) -> Add(eps) -> Sqrt -> Div(x, .) -> Mul(., w)
//   add_rmsnorm         the same on x = Add(a, b), x written out as well; b may still be split-K slabs of a MatMul
//   rope                Mul(x, cos) + Mul(Concat(Neg(x[..., D/2:]), x[..., :D/2]), sin)
//   swiglu              Mul(Mul(g, Sigmoid(g)), u)
//   scale_mask_softmax  Softmax(Add(Mul(s, scale), mask), last axis)
//
// Reference backends replaced per launch: backend/pow.rs, reduce_mean.rs, add.rs, sqrt.rs, div.rs, mul.rs;
// mul.rs, slice.rs (x2), neg.rs, concat.rs, add.rs; sigmoid.rs, mul.rs (x2); mul.rs, add.rs, softmax.rs
// (all under runtime/src/providers/cuda/backend/).
#include "common.cuh"

namespace rmlk {

__device__ __forceinline__ double warp_sum_d(double v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_sum_f(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max_f(float v) {
#pragma unroll
    for (int o = 16; o >= 1; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Optional producer of the row in front of RMSNorm: x = a + b (the residual Add of a decoder layer), where b may
// still be the `parts` split-K slabs of the MatMul that made it.  The slabs are added in slab order starting from
// 0.f, exactly as the stand-alone split-K reduction does, then a + b as the Add kernel does, and x is written to
// `sum` for the later consumers of the Add.  b == nullptr: the row is read from a as it is.
struct RowAdd {
    const float* b;
    float* sum;
    int parts;
    int64_t part_stride;
};

__device__ __forceinline__ float row_add_value(const RowAdd& r, float a, int64_t i) {
    float y;
    if (r.parts == 1) {
        y = r.b[i];
    } else {
        y = 0.f;
        for (int k = 0; k < r.parts; k++) y += r.b[k * r.part_stride + i];
    }
    return __fadd_rn(a, y);
}

// One CTA of 256 threads per row.  The squares are summed in double, as the ReduceMean kernel does.
__global__ void __launch_bounds__(256) rmsnorm_f32_kernel(int64_t cols, float exponent, float eps, const float* __restrict__ x,
                                                         const float* __restrict__ w, float* __restrict__ out, RowAdd ra) {
    dep_sync();
    __shared__ double part[8];
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * cols;
    const float* row = x + r0;
    float* dst = out + r0;
    double acc = 0.0;
    if (ra.b) {
        for (int64_t c = threadIdx.x; c < cols; c += 256) {
            const float v = row_add_value(ra, row[c], r0 + c);
            ra.sum[r0 + c] = v;
            acc += static_cast<double>(powf(v, exponent));
        }
        row = ra.sum + r0;  // each thread reads back only what it wrote itself
    } else {
        for (int64_t c = threadIdx.x; c < cols; c += 256) acc += static_cast<double>(powf(row[c], exponent));
    }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int i = 0; i < 8; i++) total += part[i];
    const float mean = static_cast<float>(total / static_cast<double>(cols));
    const float sd = sqrtf(__fadd_rn(mean, eps));
    for (int64_t c = threadIdx.x; c < cols; c += 256) dst[c] = __fmul_rn(__fdiv_rn(row[c], sd), w[c]);
}

// Same, for rows of up to THREADS * 4 * NP elements with 16-byte alignment: the row is read once and held in registers.
// A few rows (a decode step: 64) take 512 or 1024 threads with one pack each, so that the row, the residual and all
// split-K slabs of a pack are requested at once - one trip to memory instead of several; many rows take 256 threads.
template <int NP, int THREADS>
__global__ void __launch_bounds__(THREADS) rmsnorm_f32_regs_kernel(int cols, float exponent, float eps, const float* __restrict__ x,
                                                                  const float* __restrict__ w, float* __restrict__ out, RowAdd ra) {
    dep_sync();
    __shared__ double part[THREADS / 32];
    const int64_t r0 = static_cast<int64_t>(blockIdx.x) * cols;
    const float4* row = reinterpret_cast<const float4*>(x + r0);
    float4* dst = reinterpret_cast<float4*>(out + r0);
    const float4* wv = reinterpret_cast<const float4*>(w);
    const int packs = cols / 4;
    float4 v[NP];
    double acc = 0.0;
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const int c = threadIdx.x + THREADS * i;
        if (c < packs) {
            v[i] = row[c];
            if (ra.b) {
                float4 y;
                if (ra.parts == 1) {
                    y = *reinterpret_cast<const float4*>(ra.b + r0 + 4 * c);
                } else {
                    y = make_float4(0.f, 0.f, 0.f, 0.f);
                    constexpr int CH = THREADS == 512 ? 16 : 8;  // slab loads in flight, added in slab order (registers allow 16 at 512 threads)
                    for (int k0 = 0; k0 < ra.parts; k0 += CH) {
                        float4 q[CH];
#pragma unroll
                        for (int j = 0; j < CH; j++)
                            if (k0 + j < ra.parts) q[j] = *reinterpret_cast<const float4*>(ra.b + (k0 + j) * ra.part_stride + r0 + 4 * c);
#pragma unroll
                        for (int j = 0; j < CH; j++)
                            if (k0 + j < ra.parts) {
                                y.x += q[j].x; y.y += q[j].y; y.z += q[j].z; y.w += q[j].w;
                            }
                    }
                }
                v[i].x = __fadd_rn(v[i].x, y.x);
                v[i].y = __fadd_rn(v[i].y, y.y);
                v[i].z = __fadd_rn(v[i].z, y.z);
                v[i].w = __fadd_rn(v[i].w, y.w);
                *reinterpret_cast<float4*>(ra.sum + r0 + 4 * c) = v[i];
            }
            acc += static_cast<double>(powf(v[i].x, exponent));
            acc += static_cast<double>(powf(v[i].y, exponent));
            acc += static_cast<double>(powf(v[i].z, exponent));
            acc += static_cast<double>(powf(v[i].w, exponent));
        }
    }
    acc = warp_sum_d(acc);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = acc;
    __syncthreads();
    double total = 0.0;
#pragma unroll
    for (int i = 0; i < THREADS / 32; i++) total += part[i];
    const float mean = static_cast<float>(total / static_cast<double>(cols));
    const float sd = sqrtf(__fadd_rn(mean, eps));
#pragma unroll
    for (int i = 0; i < NP; i++) {
        const int c = threadIdx.x + THREADS * i;
        if (c < packs) {
            const float4 g = wv[c];
            float4 r;
            r.x = __fmul_rn(__fdiv_rn(v[i].x, sd), g.x);
            r.y = __fmul_rn(__fdiv_rn(v[i].y, sd), g.y);
            r.z = __fmul_rn(__fdiv_rn(v[i].z, sd), g.z);
            r.w = __fmul_rn(__fdiv_rn(v[i].w, sd), g.w);
            dst[c] = r;
        }
    }
}

struct RopeParams {
    int64_t d[4];         // output dims, row-major; d[3] = head dim D
    int64_t xs[4], cs[4], ss[4];  // element strides of x, cos, sin per output dim (0 = broadcast)
    int64_t os[4];                // element strides of the output (dense, or a slot inside a larger buffer)
};

__global__ void __launch_bounds__(256) rope_f32_kernel(RopeParams p, int64_t total, const float* __restrict__ x, const float* __restrict__ cosv,
                                                      const float* __restrict__ sinv, float* __restrict__ out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t D = p.d[3], half = D / 2;
    int64_t t = i;
    const int64_t j = t % D;
    t /= D;
    const int64_t i2 = t % p.d[2];
    t /= p.d[2];
    const int64_t i1 = t % p.d[1];
    const int64_t i0 = t / p.d[1];
    const int64_t xb = i0 * p.xs[0] + i1 * p.xs[1] + i2 * p.xs[2];
    const int64_t cb = i0 * p.cs[0] + i1 * p.cs[1] + i2 * p.cs[2] + j * p.cs[3];
    const int64_t sb = i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2] + j * p.ss[3];
    const float xv = x[xb + j * p.xs[3]];
    // rotate_half: Concat(Neg(x[half:]), x[:half]); Neg is x * -1
    const float rot = j < half ? __fmul_rn(x[xb + (j + half) * p.xs[3]], -1.0f) : x[xb + (j - half) * p.xs[3]];
    out[i0 * p.os[0] + i1 * p.os[1] + i2 * p.os[2] + j * p.os[3]] = __fadd_rn(__fmul_rn(xv, cosv[cb]), __fmul_rn(rot, sinv[sb]));
}

// ---- several rotary embeddings / 4-byte strided copies as one launch (blockIdx.y = job) -----------------------------------
struct BatchJob {
    int kind, rank, parts, vec;   // vec: every row is contiguous, 16-byte aligned and a multiple of 4 (rotary: of 8) long
    int64_t part_stride, total;
    int64_t threads;              // vec: 4 elements (rotary: two quads, j and j + D/2) per thread; else one element
    int64_t d[5], is[5], os[5], cs[4], ss[4];
    const float* in;
    const float* cosv;
    const float* sinv;
    float* out;
};
struct BatchParams {
    BatchJob job[RMLK_BATCH_MAX_JOBS];
};

// the value at element offset `off` of a tensor that may still be split-K slabs (added in slab order from 0.f)
__device__ __forceinline__ float batch_load(const BatchJob& j, int64_t off) {
    if (j.parts <= 1) return j.in[off];
    float s = 0.f;
    for (int k = 0; k < j.parts; k++) s += j.in[k * j.part_stride + off];
    return s;
}

// four consecutive elements at element offset `off` (16-byte aligned), slabs added in order from 0.f per component
__device__ __forceinline__ float4 batch_load4(const BatchJob& j, int64_t off) {
    if (j.parts <= 1) return *reinterpret_cast<const float4*>(j.in + off);
    float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int k = 0; k < j.parts; k++) {
        const float4 v = *reinterpret_cast<const float4*>(j.in + k * j.part_stride + off);
        s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
    }
    return s;
}

__global__ void __launch_bounds__(256) rope_copy_batch_kernel(const __grid_constant__ BatchParams bp) {
    dep_sync();
    const BatchJob& p = bp.job[blockIdx.y];
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= p.threads) return;
    if (p.vec && p.kind == RMLK_BATCH_ROPE) {
        // One thread makes outputs j .. j + 3 and j + D/2 .. j + D/2 + 3 of a head (j < D/2): both quads need x[j ..] and
        // x[j + D/2 ..], each possibly a sum of slabs, which are loaded once as 16-byte words.  Per element the expressions
        // are those of rope_f32_kernel: out[j] = x[j] cos[j] + (x[j + D/2] * -1) sin[j]; out[j + D/2] = x[j + D/2] cos[..] + x[j] sin[..].
        const int64_t half = p.d[3] / 2, quads = half / 4;
        int64_t t = i;
        const int64_t j = (t % quads) * 4;
        t /= quads;
        const int64_t i2 = t % p.d[2];
        t /= p.d[2];
        const int64_t i1 = t % p.d[1];
        const int64_t i0 = t / p.d[1];
        const int64_t xb = i0 * p.is[0] + i1 * p.is[1] + i2 * p.is[2];
        const int64_t cb = i0 * p.cs[0] + i1 * p.cs[1] + i2 * p.cs[2];
        const int64_t sb = i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2];
        const int64_t ob = i0 * p.os[0] + i1 * p.os[1] + i2 * p.os[2];
        const float4 lo = batch_load4(p, xb + j), hi = batch_load4(p, xb + j + half);
        const float4 c0 = *reinterpret_cast<const float4*>(p.cosv + cb + j), c1 = *reinterpret_cast<const float4*>(p.cosv + cb + j + half);
        const float4 s0 = *reinterpret_cast<const float4*>(p.sinv + sb + j), s1 = *reinterpret_cast<const float4*>(p.sinv + sb + j + half);
        float4 o0, o1;
        o0.x = __fadd_rn(__fmul_rn(lo.x, c0.x), __fmul_rn(__fmul_rn(hi.x, -1.0f), s0.x));
        o0.y = __fadd_rn(__fmul_rn(lo.y, c0.y), __fmul_rn(__fmul_rn(hi.y, -1.0f), s0.y));
        o0.z = __fadd_rn(__fmul_rn(lo.z, c0.z), __fmul_rn(__fmul_rn(hi.z, -1.0f), s0.z));
        o0.w = __fadd_rn(__fmul_rn(lo.w, c0.w), __fmul_rn(__fmul_rn(hi.w, -1.0f), s0.w));
        o1.x = __fadd_rn(__fmul_rn(hi.x, c1.x), __fmul_rn(lo.x, s1.x));
        o1.y = __fadd_rn(__fmul_rn(hi.y, c1.y), __fmul_rn(lo.y, s1.y));
        o1.z = __fadd_rn(__fmul_rn(hi.z, c1.z), __fmul_rn(lo.z, s1.z));
        o1.w = __fadd_rn(__fmul_rn(hi.w, c1.w), __fmul_rn(lo.w, s1.w));
        *reinterpret_cast<float4*>(p.out + ob + j) = o0;
        *reinterpret_cast<float4*>(p.out + ob + j + half) = o1;
    } else if (p.vec) {
        // copy: the innermost dim in 16-byte words
        int64_t t = i, io = 0, oo = 0;
        const int64_t quads = p.d[p.rank - 1] / 4;
        const int64_t q4 = (t % quads) * 4;
        t /= quads;
        for (int d = p.rank - 2; d >= 0; d--) {
            const int64_t q = t / p.d[d], r = t - q * p.d[d];
            io += r * p.is[d];
            oo += r * p.os[d];
            t = q;
        }
        *reinterpret_cast<float4*>(p.out + oo + q4) = batch_load4(p, io + q4);
    } else if (p.kind == RMLK_BATCH_ROPE) {
        // the expressions of rope_f32_kernel
        const int64_t D = p.d[3], half = D / 2;
        int64_t t = i;
        const int64_t j = t % D;
        t /= D;
        const int64_t i2 = t % p.d[2];
        t /= p.d[2];
        const int64_t i1 = t % p.d[1];
        const int64_t i0 = t / p.d[1];
        const int64_t xb = i0 * p.is[0] + i1 * p.is[1] + i2 * p.is[2];
        const int64_t cb = i0 * p.cs[0] + i1 * p.cs[1] + i2 * p.cs[2] + j * p.cs[3];
        const int64_t sb = i0 * p.ss[0] + i1 * p.ss[1] + i2 * p.ss[2] + j * p.ss[3];
        const float xv = batch_load(p, xb + j * p.is[3]);
        const float rot = j < half ? __fmul_rn(batch_load(p, xb + (j + half) * p.is[3]), -1.0f) : batch_load(p, xb + (j - half) * p.is[3]);
        p.out[i0 * p.os[0] + i1 * p.os[1] + i2 * p.os[2] + j * p.os[3]] = __fadd_rn(__fmul_rn(xv, p.cosv[cb]), __fmul_rn(rot, p.sinv[sb]));
    } else {
        int64_t t = i, io = 0, oo = 0;
        for (int d = p.rank - 1; d >= 0; d--) {
            const int64_t q = t / p.d[d], r = t - q * p.d[d];
            io += r * p.is[d];
            oo += r * p.os[d];
            t = q;
        }
        p.out[oo] = batch_load(p, io);
    }
}

// cos / sin tables of a rotary embedding: emb = Concat(f, f) with f = a * b, a one value per row and b one per column of f;
// cos_out, sin_out [rows, 2 half].  The same functions as the single ops (IEEE multiply, cosf, sinf), each computed once
// and written to both halves of the row.
__global__ void __launch_bounds__(256) rope_tables_kernel(int64_t total, int half, const float* __restrict__ a, const float* __restrict__ b,
                                                         float* __restrict__ cos_out, float* __restrict__ sin_out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= total) return;
    const int64_t row = i / half;
    const int j = static_cast<int>(i - row * half);
    const float f = __fmul_rn(a[row], b[j]);
    const float c = cosf(f), sn = sinf(f);
    const int64_t o = row * 2 * half + j;
    cos_out[o] = c;
    cos_out[o + half] = c;
    sin_out[o] = sn;
    sin_out[o + half] = sn;
}

// Additive attention mask of an exported decoder, [B, 1, S, T]:
//   tri = Trilu(ConstantOfShape([S, T], fill), k, upper): fill where t - s >= k, else 0
//   causal = Where(Equal(tri, cmp_tri), v_future, v_else)
//   out = Where(Equal(Cast(am -> f32), cmp_pad), v_pad, causal)          am [B, T] int64
// Only comparisons and selections of the given constants: the same bits as the seven single ops.
struct MaskChain {
    int64_t B, S, T, k;
    float fill, cmp_tri, v_future, v_else, cmp_pad, v_pad;
};
__global__ void __launch_bounds__(256) mask_chain_kernel(MaskChain p, const int64_t* __restrict__ am, float* __restrict__ out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= p.B * p.S * p.T) return;
    const int64_t t = i % p.T, s = (i / p.T) % p.S, b = i / (p.T * p.S);
    const float tri = (t - s >= p.k) ? p.fill : 0.0f;
    const float causal = (tri == p.cmp_tri) ? p.v_future : p.v_else;
    out[i] = (static_cast<float>(am[b * p.T + t]) == p.cmp_pad) ? p.v_pad : causal;
}

__global__ void __launch_bounds__(256) swiglu_f32_kernel(int64_t n, const float* __restrict__ g, const float* __restrict__ u, float* __restrict__ out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= n) return;
    const float gv = g[i];
    const float sg = 1.0f / (1.0f + expf(-gv));
    out[i] = __fmul_rn(__fmul_rn(gv, sg), u[i]);
}

__global__ void __launch_bounds__(256) swiglu_f32_vec_kernel(int64_t packs, const float4* __restrict__ g, const float4* __restrict__ u,
                                                            float4* __restrict__ out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    if (i >= packs) return;
    const float4 a = g[i], b = u[i];
    float4 r;
    r.x = __fmul_rn(__fmul_rn(a.x, 1.0f / (1.0f + expf(-a.x))), b.x);
    r.y = __fmul_rn(__fmul_rn(a.y, 1.0f / (1.0f + expf(-a.y))), b.y);
    r.z = __fmul_rn(__fmul_rn(a.z, 1.0f / (1.0f + expf(-a.z))), b.z);
    r.w = __fmul_rn(__fmul_rn(a.w, 1.0f / (1.0f + expf(-a.w))), b.w);
    out[i] = r;
}

// gate and up as [rows, cols] matrices with row pitches (columns of a wider matrix), out dense
__global__ void __launch_bounds__(256) swiglu_f32_pitched_kernel(int64_t rows, int64_t cols, const float* __restrict__ g, int64_t ldg,
                                                                const float* __restrict__ u, int64_t ldu, float* __restrict__ out) {
    dep_sync();
    const int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x;
    const int64_t packs = cols / 4;
    if (i >= rows * packs) return;
    const int64_t r = i / packs, c = (i - r * packs) * 4;
    const float4 a = *reinterpret_cast<const float4*>(g + r * ldg + c);
    const float4 b = *reinterpret_cast<const float4*>(u + r * ldu + c);
    float4 o;
    o.x = __fmul_rn(__fmul_rn(a.x, 1.0f / (1.0f + expf(-a.x))), b.x);
    o.y = __fmul_rn(__fmul_rn(a.y, 1.0f / (1.0f + expf(-a.y))), b.y);
    o.z = __fmul_rn(__fmul_rn(a.z, 1.0f / (1.0f + expf(-a.z))), b.z);
    o.w = __fmul_rn(__fmul_rn(a.w, 1.0f / (1.0f + expf(-a.w))), b.w);
    *reinterpret_cast<float4*>(out + r * cols + c) = o;
}

struct MaskParams {
    int64_t d[3];   // leading dims of the scores [d0, d1, d2, cols]
    int64_t ms[3];  // mask element strides for those dims (0 = broadcast); mask rows are dense
};

// One warp per row of up to 32 * PER columns, the row held in registers.
template <int PER>
__global__ void __launch_bounds__(256) scale_mask_softmax_f32_kernel(MaskParams p, int64_t rows, int cols, float scale, const float* __restrict__ s,
                                                                    const float* __restrict__ mask, float* __restrict__ out) {
    dep_sync();
    const int64_t row = (static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x) >> 5;
    if (row >= rows) return;
    const int lane = threadIdx.x & 31;
    int64_t t = row;
    const int64_t i2 = t % p.d[2];
    t /= p.d[2];
    const int64_t i1 = t % p.d[1];
    const int64_t i0 = t / p.d[1];
    const float* src = s + row * cols;
    const float* mrow = mask + i0 * p.ms[0] + i1 * p.ms[1] + i2 * p.ms[2];
    float v[PER];
    float mx = -INFINITY;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        const int c = lane + 32 * k;
        v[k] = -INFINITY;
        if (c < cols) {
            v[k] = __fadd_rn(__fmul_rn(src[c], scale), mrow[c]);
            mx = fmaxf(mx, v[k]);
        }
    }
    mx = warp_max_f(mx);
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        const int c = lane + 32 * k;
        if (c < cols) {
            v[k] = expf(v[k] - mx);
            sum += v[k];
        }
    }
    sum = warp_sum_f(sum);
    float* dst = out + row * cols;
#pragma unroll
    for (int k = 0; k < PER; k++) {
        const int c = lane + 32 * k;
        if (c < cols) dst[c] = v[k] / sum;
    }
}

}  // namespace rmlk

using namespace rmlk;

static int launch_rmsnorm(rmlk_stream_t stream, int64_t rows, int64_t cols, const void* x, float exponent, float eps, const void* weight,
                          void* out, const RowAdd& ra) {
    const float* xp = static_cast<const float*>(x);
    const float* wp = static_cast<const float*>(weight);
    float* op = static_cast<float*>(out);
    cudaStream_t st = as_stream(stream);
    const unsigned grid = static_cast<unsigned>(rows);
    const bool add_ok = !ra.b || (aligned_to(ra.b, 16) && aligned_to(ra.sum, 16) && ra.part_stride % 4 == 0);
    if (cols % 4 == 0 && cols <= 4096 && aligned_to(x, 16) && aligned_to(weight, 16) && aligned_to(out, 16) && add_ok) {
        const int c = static_cast<int>(cols);
        const bool few = rows <= 512;  // too few rows to fill the GPU with 256-thread CTAs: widen the CTA instead
        if (cols <= 1024) launch_dep(rmsnorm_f32_regs_kernel<1, 256>, dim3(grid), dim3(256), 0, st, c, exponent, eps, xp, wp, op, ra);
        else if (cols <= 2048 && few) launch_dep(rmsnorm_f32_regs_kernel<1, 512>, dim3(grid), dim3(512), 0, st, c, exponent, eps, xp, wp, op, ra);
        else if (cols <= 2048) launch_dep(rmsnorm_f32_regs_kernel<2, 256>, dim3(grid), dim3(256), 0, st, c, exponent, eps, xp, wp, op, ra);
        else if (few) launch_dep(rmsnorm_f32_regs_kernel<1, 1024>, dim3(grid), dim3(1024), 0, st, c, exponent, eps, xp, wp, op, ra);
        else launch_dep(rmsnorm_f32_regs_kernel<4, 256>, dim3(grid), dim3(256), 0, st, c, exponent, eps, xp, wp, op, ra);
    } else {
        launch_dep(rmsnorm_f32_kernel, dim3(grid), dim3(256), 0, st, cols, exponent, eps, xp, wp, op, ra);
    }
    RMLK_CHECK_LAUNCH("rmsnorm_f32_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_rmsnorm(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* x, float exponent, float eps,
                                 const void* weight, void* out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for rmsnorm (f32 only)");
    if (rows < 0 || cols < 0) return fail(RMLK_ERR_INVALID_ARG, "rmsnorm: negative extent");
    if (rows == 0 || cols == 0) return RMLK_OK;
    if (!x || !weight || !out) return fail(RMLK_ERR_INVALID_ARG, "rmsnorm: NULL tensor pointer");
    if (rows > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "rmsnorm: too many rows");
    RowAdd ra = {nullptr, nullptr, 0, 0};
    return launch_rmsnorm(stream, rows, cols, x, exponent, eps, weight, out, ra);
}

extern "C" int rmlk_b200_add_rmsnorm(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* a, const void* b, int b_parts,
                                     int64_t b_part_stride, float exponent, float eps, const void* weight, void* sum_out, void* norm_out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for add_rmsnorm (f32 only)");
    if (rows < 0 || cols < 0) return fail(RMLK_ERR_INVALID_ARG, "add_rmsnorm: negative extent");
    if (b_parts < 1 || b_parts > 64) return fail(RMLK_ERR_INVALID_ARG, "add_rmsnorm: b_parts must be 1..64");
    if (b_parts > 1 && b_part_stride < rows * cols) return fail(RMLK_ERR_INVALID_ARG, "add_rmsnorm: slabs of b overlap");
    if (rows == 0 || cols == 0) return RMLK_OK;
    if (!a || !b || !weight || !sum_out || !norm_out) return fail(RMLK_ERR_INVALID_ARG, "add_rmsnorm: NULL tensor pointer");
    if (rows > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "add_rmsnorm: too many rows");
    RowAdd ra = {static_cast<const float*>(b), static_cast<float*>(sum_out), b_parts, b_part_stride};
    return launch_rmsnorm(stream, rows, cols, a, exponent, eps, weight, norm_out, ra);
}

extern "C" int rmlk_b200_rope(rmlk_stream_t stream, int dtype, const int64_t* shape4, const int64_t* x_strides, const int64_t* cos_strides,
                              const int64_t* sin_strides, const void* x, const void* cosv, const void* sinv, void* out) {
    return rmlk_b200_rope_to(stream, dtype, shape4, x_strides, cos_strides, sin_strides, x, cosv, sinv, out, nullptr);
}

extern "C" int rmlk_b200_rope_to(rmlk_stream_t stream, int dtype, const int64_t* shape4, const int64_t* x_strides, const int64_t* cos_strides,
                                 const int64_t* sin_strides, const void* x, const void* cosv, const void* sinv, void* out,
                                 const int64_t* out_strides) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for rope (f32 only)");
    if (!shape4 || !x_strides || !cos_strides || !sin_strides) return fail(RMLK_ERR_INVALID_ARG, "rope: NULL shape / strides");
    RopeParams p;
    int64_t total = 1;
    for (int d = 0; d < 4; d++) {
        if (shape4[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "rope: negative extent");
        p.d[d] = shape4[d];
        p.xs[d] = x_strides[d];
        p.cs[d] = cos_strides[d];
        p.ss[d] = sin_strides[d];
        total *= shape4[d];
    }
    int64_t run = 1;
    for (int d = 3; d >= 0; d--) {  // dense output unless the caller places it
        p.os[d] = out_strides ? out_strides[d] : run;
        run *= shape4[d] > 0 ? shape4[d] : 1;
    }
    if (total == 0) return RMLK_OK;
    if (shape4[3] % 2) return fail(RMLK_ERR_INVALID_ARG, "rope: head dim must be even");
    if (!x || !cosv || !sinv || !out) return fail(RMLK_ERR_INVALID_ARG, "rope: NULL tensor pointer");
    if (ceil_div64(total, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "rope: tensor too large");
    launch_dep(rope_f32_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, as_stream(stream), 
        p, total, static_cast<const float*>(x), static_cast<const float*>(cosv), static_cast<const float*>(sinv), static_cast<float*>(out));
    RMLK_CHECK_LAUNCH("rope_f32_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_causal_padding_mask(rmlk_stream_t stream, int64_t batch, int64_t s_len, int64_t t_len, int64_t k, const void* attention_mask,
                                             float fill, float cmp_tri, float v_future, float v_else, float cmp_pad, float v_pad, void* out) {
    if (batch < 0 || s_len < 0 || t_len < 0) return fail(RMLK_ERR_INVALID_ARG, "causal_padding_mask: negative extent");
    const int64_t total = batch * s_len * t_len;
    if (total == 0) return RMLK_OK;
    if (!attention_mask || !out) return fail(RMLK_ERR_INVALID_ARG, "causal_padding_mask: NULL tensor pointer");
    if (ceil_div64(total, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "causal_padding_mask: tensor too large");
    MaskChain p = {batch, s_len, t_len, k, fill, cmp_tri, v_future, v_else, cmp_pad, v_pad};
    launch_dep(mask_chain_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, as_stream(stream), p,
               static_cast<const int64_t*>(attention_mask), static_cast<float*>(out));
    RMLK_CHECK_LAUNCH("mask_chain_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_rope_tables(rmlk_stream_t stream, int dtype, int64_t rows, int64_t half, const void* a, const void* b, void* cos_out,
                                     void* sin_out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for rope_tables (f32 only)");
    if (rows < 0 || half < 0 || half > 0x3fffffffll) return fail(RMLK_ERR_INVALID_ARG, "rope_tables: bad extent");
    if (rows == 0 || half == 0) return RMLK_OK;
    if (!a || !b || !cos_out || !sin_out) return fail(RMLK_ERR_INVALID_ARG, "rope_tables: NULL tensor pointer");
    const int64_t total = rows * half;
    if (ceil_div64(total, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "rope_tables: tensor too large");
    launch_dep(rope_tables_kernel, dim3(static_cast<unsigned>(ceil_div64(total, 256))), dim3(256), 0, as_stream(stream), total, static_cast<int>(half),
               static_cast<const float*>(a), static_cast<const float*>(b), static_cast<float*>(cos_out), static_cast<float*>(sin_out));
    RMLK_CHECK_LAUNCH("rope_tables_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_rope_copy_batch(rmlk_stream_t stream, int n_jobs, const rmlk_batch_job* jobs) {
    if (n_jobs < 0 || n_jobs > RMLK_BATCH_MAX_JOBS) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: between 0 and 4 jobs");
    if (n_jobs == 0) return RMLK_OK;
    if (!jobs) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: NULL jobs");
    BatchParams bp;
    int n = 0;
    int64_t most = 0;
    for (int q = 0; q < n_jobs; q++) {
        const rmlk_batch_job& src = jobs[q];
        if (src.kind != RMLK_BATCH_ROPE && src.kind != RMLK_BATCH_COPY4) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: unknown job kind");
        const int rank = src.kind == RMLK_BATCH_ROPE ? 4 : src.rank;
        if (rank < 1 || rank > 5) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: rank must be 1..5 (4 for a rotary job)");
        BatchJob& j = bp.job[n];
        j.kind = src.kind;
        j.rank = rank;
        j.parts = src.in_parts > 1 ? src.in_parts : 1;
        j.vec = 0;
        j.part_stride = src.in_part_stride;
        j.total = 1;
        for (int d = 0; d < 5; d++) {
            j.d[d] = d < rank ? src.shape[d] : 1;
            j.is[d] = d < rank ? src.in_strides[d] : 0;
            j.os[d] = d < rank ? src.out_strides[d] : 0;
            if (j.d[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: negative extent");
            j.total *= j.d[d];
        }
        for (int d = 0; d < 4; d++) {
            j.cs[d] = src.cos_strides[d];
            j.ss[d] = src.sin_strides[d];
        }
        if (j.total == 0) continue;
        if (src.kind == RMLK_BATCH_ROPE && (j.d[3] % 2)) return fail(RMLK_ERR_INVALID_ARG, "rope: head dim must be even");
        if (!src.in || !src.out || (src.kind == RMLK_BATCH_ROPE && (!src.cosv || !src.sinv)))
            return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: NULL tensor pointer");
        if (ceil_div64(j.total, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "rope_copy_batch: tensor too large");
        j.in = static_cast<const float*>(src.in);
        j.cosv = static_cast<const float*>(src.cosv);
        j.sinv = static_cast<const float*>(src.sinv);
        j.out = static_cast<float*>(src.out);
        // 16-byte form: contiguous innermost dim on every tensor, all other strides and the bases multiples of 4 elements
        static const bool vec_ok = [] {
            const char* e = getenv("RMLK_B200_NO_BATCH_VEC");
            return !(e && e[0] == '1');
        }();
        bool vec = vec_ok && j.d[rank - 1] % (src.kind == RMLK_BATCH_ROPE ? 8 : 4) == 0 && j.is[rank - 1] == 1 && j.os[rank - 1] == 1 &&
                   aligned_to(src.in, 16) && aligned_to(src.out, 16) && j.part_stride % 4 == 0;
        for (int d = 0; d < rank - 1 && vec; d++) vec = j.is[d] % 4 == 0 && j.os[d] % 4 == 0;
        if (src.kind == RMLK_BATCH_ROPE && vec) {
            vec = j.cs[3] == 1 && j.ss[3] == 1 && aligned_to(src.cosv, 16) && aligned_to(src.sinv, 16);
            for (int d = 0; d < 3 && vec; d++) vec = j.cs[d] % 4 == 0 && j.ss[d] % 4 == 0;
        }
        j.vec = vec ? 1 : 0;
        j.threads = !vec ? j.total : src.kind == RMLK_BATCH_ROPE ? j.total / 8 : j.total / 4;
        if (j.threads > most) most = j.threads;
        n++;
    }
    if (n == 0) return RMLK_OK;
    for (int q = n; q < RMLK_BATCH_MAX_JOBS; q++) {
        bp.job[q] = bp.job[0];
        bp.job[q].total = 0;
        bp.job[q].threads = 0;
    }
    launch_dep(rope_copy_batch_kernel, dim3(static_cast<unsigned>(ceil_div64(most, 256)), static_cast<unsigned>(n)), dim3(256), 0, as_stream(stream), bp);
    RMLK_CHECK_LAUNCH("rope_copy_batch_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_swiglu(rmlk_stream_t stream, int dtype, int64_t n, const void* gate, const void* up, void* out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for swiglu (f32 only)");
    if (n < 0) return fail(RMLK_ERR_INVALID_ARG, "swiglu: negative extent");
    if (n == 0) return RMLK_OK;
    if (!gate || !up || !out) return fail(RMLK_ERR_INVALID_ARG, "swiglu: NULL tensor pointer");
    cudaStream_t st = as_stream(stream);
    if (n % 4 == 0 && aligned_to(gate, 16) && aligned_to(up, 16) && aligned_to(out, 16) && ceil_div64(n / 4, 256) <= 0x7fffffffll) {
        launch_dep(swiglu_f32_vec_kernel, dim3(static_cast<unsigned>(ceil_div64(n / 4, 256))), dim3(256), 0, st, n / 4, static_cast<const float4*>(gate),
                                                                                             static_cast<const float4*>(up), static_cast<float4*>(out));
    } else {
        if (ceil_div64(n, 256) > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "swiglu: tensor too large");
        launch_dep(swiglu_f32_kernel, dim3(static_cast<unsigned>(ceil_div64(n, 256))), dim3(256), 0, st, n, static_cast<const float*>(gate), static_cast<const float*>(up),
                                                                                     static_cast<float*>(out));
    }
    RMLK_CHECK_LAUNCH("swiglu_f32_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_swiglu_pitched(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* gate, int64_t gate_pitch,
                                        const void* up, int64_t up_pitch, void* out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for swiglu (f32 only)");
    if (rows < 0 || cols < 0) return fail(RMLK_ERR_INVALID_ARG, "swiglu: negative extent");
    if (rows == 0 || cols == 0) return RMLK_OK;
    if (!gate || !up || !out) return fail(RMLK_ERR_INVALID_ARG, "swiglu: NULL tensor pointer");
    if (cols % 4 || gate_pitch % 4 || up_pitch % 4 || !aligned_to(gate, 16) || !aligned_to(up, 16) || !aligned_to(out, 16))
        return fail(RMLK_ERR_INVALID_ARG, "swiglu_pitched: columns, pitches and pointers must be multiples of 4 elements / 16 bytes");
    const int64_t blocks = ceil_div64(rows * (cols / 4), 256);
    if (blocks > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "swiglu: tensor too large");
    launch_dep(swiglu_f32_pitched_kernel, dim3(static_cast<unsigned>(blocks)), dim3(256), 0, as_stream(stream), rows, cols, static_cast<const float*>(gate), gate_pitch,
                                                                                            static_cast<const float*>(up), up_pitch, static_cast<float*>(out));
    RMLK_CHECK_LAUNCH("swiglu_f32_pitched_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_scale_mask_softmax(rmlk_stream_t stream, int dtype, const int64_t* lead3, int64_t cols, const int64_t* mask_strides3,
                                            float scale, const void* scores, const void* mask, void* out) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for scale_mask_softmax (f32 only)");
    if (!lead3 || !mask_strides3) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: NULL dims / strides");
    MaskParams p;
    int64_t rows = 1;
    for (int d = 0; d < 3; d++) {
        if (lead3[d] < 0) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: negative extent");
        p.d[d] = lead3[d];
        p.ms[d] = mask_strides3[d];
        rows *= lead3[d];
    }
    if (cols < 0) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: negative extent");
    if (rows == 0 || cols == 0) return RMLK_OK;
    if (cols > 2048) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: rows longer than 2048 are not supported");
    if (!scores || !mask || !out) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: NULL tensor pointer");
    const int64_t blocks = ceil_div64(rows, 8);
    if (blocks > 0x7fffffffll) return fail(RMLK_ERR_INVALID_ARG, "scale_mask_softmax: too many rows");
    cudaStream_t st = as_stream(stream);
    const float* s = static_cast<const float*>(scores);
    const float* m = static_cast<const float*>(mask);
    float* o = static_cast<float*>(out);
    const unsigned grid = static_cast<unsigned>(blocks);
    const int c = static_cast<int>(cols);
    if (cols <= 128) launch_dep(scale_mask_softmax_f32_kernel<4>, dim3(grid), dim3(256), 0, st, p, rows, c, scale, s, m, o);
    else if (cols <= 256) launch_dep(scale_mask_softmax_f32_kernel<8>, dim3(grid), dim3(256), 0, st, p, rows, c, scale, s, m, o);
    else if (cols <= 512) launch_dep(scale_mask_softmax_f32_kernel<16>, dim3(grid), dim3(256), 0, st, p, rows, c, scale, s, m, o);
    else if (cols <= 1024) launch_dep(scale_mask_softmax_f32_kernel<32>, dim3(grid), dim3(256), 0, st, p, rows, c, scale, s, m, o);
    else launch_dep(scale_mask_softmax_f32_kernel<64>, dim3(grid), dim3(256), 0, st, p, rows, c, scale, s, m, o);
    RMLK_CHECK_LAUNCH("scale_mask_softmax_f32_kernel");
    return RMLK_OK;
}
