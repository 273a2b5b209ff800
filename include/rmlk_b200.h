/*
 * rmlk_b200 — B200 (sm_100a) operator kernels behind a C ABI.
 *
 * This header is the drop-in boundary for the reference project's `cuda` crate: every entry point
 * below replaces the body of one launch wrapper in the reference's cuda/src/kernels/<op>.rs (cited
 * per function), or one of the host-side memcpy / library paths in
 * runtime/src/providers/cuda/backend/<op>.rs for the ops that have no kernel there.
 *
 * Conventions
 *  - All tensor pointers are DEVICE pointers to dense row-major buffers owned by the caller; the
 *    library never allocates, frees or retains them.  Shapes, strides, axes, perms and scalar
 *    parameters are HOST values passed by value or as small host arrays; nothing is read back
 *    from the device, so no entry point synchronises the stream.
 *  - Strides are in ELEMENTS; a stride of 0 broadcasts that dimension (the reference's
 *    runtime/src/utils/mod.rs:56-111 convention).  Rank is at most RMLK_MAX_RANK.  A scalar is
 *    passed the way the reference passes it to kernels: rank 1, shape {1}
 *    (runtime/src/providers/cuda/utils.rs:5-18).
 *  - `stream` is a cudaStream_t (NULL = legacy default stream).  Work is enqueued on it and the
 *    call returns.  Entry points may be called from several threads (one per GPU, or several per GPU on
 *    different streams).  The only process-wide state is a set of lazily filled, write-once caches: the SM
 *    count per device, the driver's tensor-map encoder, per-device "kernel configured" flags
 *    (cudaFuncSetAttribute for kernels that need more than 48 KB of shared memory), the address of the
 *    built-in scratch of rmlk_b200_matmul_static, and the environment switches read at first use.  They are
 *    published with atomics / std::call_once, so concurrent first calls are safe.  The first call of a kernel
 *    family on a device therefore does a little more host work than later ones (and should come before any
 *    stream capture).
 *  - Return value: RMLK_OK, an RMLK_ERR_* code, or RMLK_ERR_CUDA_BASE + cudaError_t.  Nothing
 *    aborts or traps.  Kernels that can meet bad data (Gather / ScatterND indices) report through
 *    a caller-provided device status word, as the reference's ScatterND does
 *    (cuda/src/ptx/headers/scatter_op_macros.cuh:56-63, :82-85).
 *  - rmlk_b200_last_error() returns a thread-local, human-readable message for the last non-OK
 *    return on the calling thread.
 */
#ifndef RMLK_B200_H
#define RMLK_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define RMLK_MAX_RANK 8

#if defined(__GNUC__)
#define RMLK_API __attribute__((visibility("default")))
#else
#define RMLK_API
#endif

typedef void* rmlk_stream_t;

/* Discriminants follow rmlk_schema::DataType's declaration order (schema/src/tensor.rs:347-375). */
typedef enum {
    RMLK_F16 = 0,
    RMLK_F32 = 1,
    RMLK_F64 = 2,
    RMLK_I32 = 3,
    RMLK_I64 = 4,
    RMLK_UNDEFINED = 5,
    RMLK_U8 = 6,
    RMLK_I8 = 7,
    RMLK_U16 = 8,
    RMLK_I16 = 9,
    RMLK_U32 = 10,
    RMLK_U64 = 11,
    RMLK_STRING = 12,
    RMLK_BOOL = 13
} rmlk_dtype;

/* Mirrors rmlk_cuda::Error (cuda/src/error.rs:6-14). */
typedef enum {
    RMLK_OK = 0,
    RMLK_ERR_INVALID_ARG = 1,       /* Error::InvalidArguments     */
    RMLK_ERR_UNSUPPORTED_DTYPE = 2, /* UnsupportedDataType (runtime/src/core/error.rs:4-10) */
    RMLK_ERR_NOT_CONTIGUOUS = 3,    /* Error::NonContiguousMemory  */
    RMLK_ERR_INTERNAL = 4,          /* Error::Internal             */
    RMLK_ERR_TIMEOUT = 5,
    RMLK_ERR_KERNEL_STATUS = 6,     /* a device status word was non-zero (ScatterNdError::KernelFailed) */
    RMLK_ERR_CUDA_BASE = 1000       /* + cudaError_t: Error::Cuda(code) */
} rmlk_status;

typedef enum {
    RMLK_BIN_ADD = 0,
    RMLK_BIN_SUB = 1,
    RMLK_BIN_MUL = 2,
    RMLK_BIN_DIV = 3,
    RMLK_BIN_EQUAL = 4,  /* output dtype bool */
    RMLK_BIN_GREATER = 5 /* output dtype bool */
} rmlk_binary_op;

typedef enum {
    RMLK_UN_SQRT = 0,
    RMLK_UN_NEG = 1,
    RMLK_UN_SIN = 2,
    RMLK_UN_COS = 3,
    RMLK_UN_SIGMOID = 4,
    RMLK_UN_RELU = 5
} rmlk_unary_op;

typedef enum {
    RMLK_SCATTER_NONE = 0,
    RMLK_SCATTER_ADD = 1,
    RMLK_SCATTER_MUL = 2,
    RMLK_SCATTER_MAX = 3,
    RMLK_SCATTER_MIN = 4
} rmlk_scatter_reduction;

RMLK_API const char* rmlk_b200_last_error(void);
RMLK_API const char* rmlk_b200_version(void);
RMLK_API size_t rmlk_b200_dtype_size(int dtype);

/* Add / Sub / Mul / Div / Equal / Greater with two-way broadcasting.
 * Replaces rmlk_cuda::kernels::binary::compute_with_types (cuda/src/kernels/binary.rs:58-100) and
 * the kernels {add,sub,mul,div,equal,greater}_fwd_* (cuda/src/ptx/headers/binary_op_macros.cuh:14-42).
 * `shape` is the output shape; dtype in {f16,f32,f64,i32,i64}; Equal/Greater write 1-byte bools. */
RMLK_API int rmlk_b200_binary(rmlk_stream_t stream, int op, int dtype, int rank, const int64_t* shape,
                     const int64_t* a_strides, const int64_t* b_strides, const void* a, const void* b, void* out);

/* Pow with independent base / exponent dtypes, output dtype = base dtype.
 * Replaces rmlk_cuda::kernels::pow::compute (cuda/src/kernels/pow.rs:140-184), kernels
 * pow_fwd_<base>_<exp> (cuda/src/ptx/pow.cu:6-65): base in {f16,f32,f64,i32,i64}, exponent in
 * {u8,u16,u32,u64,i8,i16,i32,i64,f16,f32,f64}. */
RMLK_API int rmlk_b200_pow(rmlk_stream_t stream, int base_dtype, int exp_dtype, int rank, const int64_t* shape,
                  const int64_t* a_strides, const int64_t* b_strides, const void* base, const void* exponent,
                  void* out);

/* Sqrt / Neg / Sin / Cos over a contiguous buffer: replaces rmlk_cuda::kernels::unary::compute
 * (cuda/src/kernels/unary.rs:10-42; kernels sqrt.cu, neg.cu, sin.cu, cos.cu).  Sigmoid / Relu replace
 * rmlk_cuda::kernels::sigmoid::compute / relu::compute (cuda/src/kernels/activation.rs:6-39), which
 * call cudnnActivationForward.  Float ops take {f16,f32,f64}; Neg and Relu also {i32,i64}. */
RMLK_API int rmlk_b200_unary(rmlk_stream_t stream, int op, int dtype, size_t n, const void* in, void* out);

/* Cast over a contiguous buffer: replaces rmlk_cuda::kernels::unary::explicit_io_types_compute
 * (cuda/src/kernels/unary.rs:47-80; kernels cast_fwd_<src>_to_<dst>, cuda/src/ptx/cast.cu:6-124).
 * Every pair over {f16,f32,f64,i8,u8,i16,u16,i32,u32,i64,u64,bool} is accepted. */
RMLK_API int rmlk_b200_cast(rmlk_stream_t stream, int src_dtype, int dst_dtype, size_t n, const void* in, void* out);

/* Where with three-way broadcasting: replaces rmlk_cuda::kernels::whereop::compute
 * (cuda/src/kernels/whereop.rs:57-101; kernels where_fwd_*, cuda/src/ptx/headers/ternary_op_macro.cuh:1-34).
 * `cond` is a 1-byte bool tensor; dtype (of x, y, out) in {f16,f32,f64,i32,i64}. */
RMLK_API int rmlk_b200_where(rmlk_stream_t stream, int dtype, int rank, const int64_t* shape, const int64_t* x_strides,
                    const int64_t* y_strides, const int64_t* cond_strides, const void* x, const void* y,
                    const void* cond, void* out);

/* ReduceMean over `axes` of a dense row-major input: replaces rmlk_cuda::kernels::reduce_mean::compute
 * (cuda/src/kernels/reduce_mean.rs:40-93; kernels reduce_mean_fwd_*,
 * cuda/src/ptx/headers/aggregation_op_macros.cuh:1-49).  Axes are normalised (0 <= axis < rank),
 * unique, in any order.  The output is dense with the reduced dims removed or kept as 1 (same
 * buffer either way).  dtype in {f16,f32,f64,i32,i64}; integers use the reference's unsigned
 * accumulate (cuda/src/ptx/reduce_mean.cu:8-9). */
RMLK_API int rmlk_b200_reduce_mean(rmlk_stream_t stream, int dtype, int rank, const int64_t* shape, int num_axes,
                          const int64_t* axes, const void* in, void* out);

/* Softmax over the last dimension of a [rows, cols] view: replaces rmlk_cuda::kernels::softmax::compute
 * (cuda/src/kernels/softmax.rs:5-37, cudnnSoftmaxForward MODE_CHANNEL on [N,C,1,1]).  dtype f32 (the
 * only one the reference dispatches, backend/softmax.rs:114-117), plus f16/f64. */
RMLK_API int rmlk_b200_softmax(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* in, void* out);

/* Softmax over the middle dimension of an [outer, channels, inner] view — the reference's second
 * accepted form, axis 1 of a rank-4 tensor in cuDNN's MODE_CHANNEL (backend/softmax.rs:45-50). f32. */
RMLK_API int rmlk_b200_softmax_strided(rmlk_stream_t stream, int dtype, int64_t outer, int64_t channels, int64_t inner,
                                       const void* in, void* out);

/* Gather along one axis of data viewed as [outer, axis_dim, inner]; out is [outer, n_idx, inner].
 * Replaces the host loop of cuMemcpyDtoD calls in runtime/src/providers/cuda/backend/gather.rs:199-258
 * (indices stay on the device; no D2H copy).  idx_dtype in {i32,i64}; negative indices wrap once.
 * An index outside [-axis_dim, axis_dim) writes 1 to *status (if non-NULL) and the row is skipped. */
RMLK_API int rmlk_b200_gather(rmlk_stream_t stream, int elem_size, int idx_dtype, int64_t outer, int64_t axis_dim,
                     int64_t inner, int64_t n_idx, const void* data, const void* indices, void* out, int* status);

/* ScatterND: out = data, then out[indices[t]] (op)= updates[t] for each index tuple t.
 * Replaces rmlk_cuda::kernels::scatter_nd::compute (cuda/src/kernels/scatter_nd.rs:91-174; kernels
 * scatter_nd{,_add,_mul,_max,_min}_fwd_*, cuda/src/ptx/headers/scatter_op_macros.cuh:19-93) and the
 * data -> output copy of backend/scatter_nd.rs:128-129 (skipped when data == out).
 * data is [data_shape...]; indices is [n_tuples, k] int64; updates is [n_tuples, slice_len] where
 * slice_len = prod(data_shape[k:]).  *status (device int, zeroed by the caller) receives 1 for an
 * index outside [-dim, dim), as the reference's `error` word does. */
RMLK_API int rmlk_b200_scatter_nd(rmlk_stream_t stream, int reduction, int dtype, int data_rank, const int64_t* data_shape,
                         int64_t n_tuples, int k, const void* data, const void* indices, const void* updates,
                         void* out, int* status);

/* Host helper: ONNX Slice normalisation.  Fills, per input axis, the clamped start, the step and the
 * output extent.  Same arithmetic as runtime/src/providers/cuda/backend/slice.rs:358-464
 * (compute_output_shape_helper) and the in-kernel copy of it,
 * cuda/src/ptx/headers/slice_op_macros.cuh:24-75.  axes / steps may be NULL. */
RMLK_API int rmlk_b200_slice_params(int rank, const int64_t* in_shape, int n, const int64_t* starts, const int64_t* ends,
                           const int64_t* axes, const int64_t* steps, int64_t* out_starts, int64_t* out_steps,
                           int64_t* out_shape);

/* Slice with per-axis normalised start / step (from rmlk_b200_slice_params):
 * out[i0,..] = in[start0 + step0*i0, ..].  Replaces rmlk_cuda::kernels::slice::compute
 * (cuda/src/kernels/slice.rs:61-122; kernels slice_fwd_*_with_index_*). */
RMLK_API int rmlk_b200_slice(rmlk_stream_t stream, int elem_size, int rank, const int64_t* in_shape,
                    const int64_t* out_shape, const int64_t* starts, const int64_t* steps, const void* in,
                    void* out);

/* Transpose: out.shape[d] = in.shape[perm[d]].  Replaces rmlk_cuda::kernels::transpose::compute
 * (cuda/src/kernels/transpose.rs:38-80; kernels transpose_fwd_*). */
RMLK_API int rmlk_b200_transpose(rmlk_stream_t stream, int elem_size, int rank, const int64_t* in_shape,
                        const int64_t* perm, const void* in, void* out);

/* Dense row-major copy of a strided view: out[i0,..] = in[sum_d i_d * strides[d]] (strides in elements; 0
 * broadcasts a dim).  One launch replaces a chain of the reference's copying layout ops - Expand
 * (cuda/src/kernels/expand.rs:35-76) followed by Reshape (a copy there, backend/reshape.rs) and Transpose
 * (cuda/src/kernels/transpose.rs:38-80) - when the host runtime has kept the chain as a view. */
RMLK_API int rmlk_b200_strided_copy(rmlk_stream_t stream, int elem_size, int rank, const int64_t* shape,
                           const int64_t* strides, const void* in, void* out);
/* Strided view -> strided view in one launch: element i (row-major over `shape`) is read at sum idx_d * in_strides[d]
 * and written at sum idx_d * out_strides[d] (strides in elements; the views must not overlap; fewer than 2^31 units).
 * Used to put rows that exist only as a view straight into their slot of a carried cache, where the reference runs
 * Transpose (backend/transpose.rs:44-178) and then Concat over the whole cache (backend/concat.rs:28-198). */
RMLK_API int rmlk_b200_strided_copy_to(rmlk_stream_t stream, int elem_size, int rank, const int64_t* shape, const int64_t* in_strides,
                              const int64_t* out_strides, const void* in, void* out);

/* Concat of n_inputs tensors along an axis; every input is viewed as [outer, axis_dims[i] * inner].
 * Replaces the nested cuMemcpyDtoD loops of runtime/src/providers/cuda/backend/concat.rs:28-76.
 * Zero-length inputs are allowed. */
RMLK_API int rmlk_b200_concat(rmlk_stream_t stream, int elem_size, int n_inputs, int64_t outer, int64_t inner,
                     const int64_t* axis_dims, const void* const* inputs, void* out);

/* Expand (right-aligned broadcast copy): replaces rmlk_cuda::kernels::expand::compute
 * (cuda/src/kernels/expand.rs:35-76; kernels expand_fwd_*). */
RMLK_API int rmlk_b200_expand(rmlk_stream_t stream, int elem_size, int in_rank, const int64_t* in_shape, int out_rank,
                     const int64_t* out_shape, const void* in, void* out);

/* Trilu on a [batch, rows, cols] view: replaces rmlk_cuda::kernels::trilu::compute
 * (cuda/src/kernels/trilu.rs:36-78; kernels trilu_fwd_*).  Masked elements are written as zero. */
RMLK_API int rmlk_b200_trilu(rmlk_stream_t stream, int elem_size, int64_t batch, int64_t rows, int64_t cols, int upper,
                    int64_t k, const void* in, void* out);

/* Range: out[i] = start + (T)i * delta for i < n, evaluated in T with two roundings, as the host loop
 * of runtime/src/providers/cuda/backend/range.rs:195-205 does.  `start` / `delta` point to HOST scalars
 * of `dtype` in {f16,f32,f64,i32,i64}. */
RMLK_API int rmlk_b200_range(rmlk_stream_t stream, int dtype, int64_t n, const void* start, const void* delta, void* out);

/* Fill a contiguous buffer with one value (`value` points to a HOST scalar of elem_size bytes).
 * Replaces the host fill + H2D copy of runtime/src/providers/cuda/backend/constant_of_shape.rs:59-62. */
RMLK_API int rmlk_b200_fill(rmlk_stream_t stream, int elem_size, int64_t n, const void* value, void* out);

/* Writes up to 32 eight-byte words, passed by value from HOST memory, to device memory with a
 * one-block kernel (no copy-engine round trip).  Used for Shape outputs and other tiny host-computed
 * tensors that the reference uploads with a synchronous memcpy_htod (backend/shape.rs:67-72). */
RMLK_API int rmlk_b200_store_small(rmlk_stream_t stream, int n_words, const uint64_t* words, void* out);

/* Batched row-major MatMul, C[b] = A[b] x B[b], fp32 accumulate:
 * replaces rmlk_cuda::kernels::gemm::compute (cuda/src/kernels/gemm.rs:112-232,
 * cublasGemmStridedBatchedEx).  A is [m,k], B is [k,n], C is [m,n], each dense; batch strides are in
 * elements and may be 0 to broadcast an operand over the batch (the reference materialises copies,
 * backend/matmul.rs:48-86).  dtype f32, or f16 (half in and out, fp32 accumulation - the reference asks cuBLAS
 * for CUBLAS_COMPUTE_16F there, cuda/src/params.rs:24-31; SIMT kernel, no workspace).  `workspace` is optional caller-owned device scratch of
 * `workspace_bytes` (see rmlk_b200_matmul_workspace_bytes); NULL selects kernels that need none. */
/* rmlk_b200_matmul passes no status word: should a bounded wait inside the tensor-core kernel ever expire (it
 * never has on a healthy device), the affected tiles of C are left unwritten and the call still returns RMLK_OK -
 * callers that must detect this use rmlk_b200_matmul_ex with a status word. */
RMLK_API int rmlk_b200_matmul(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                     const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                     int64_t c_batch_stride, void* workspace, size_t workspace_bytes);
/* Same, with a device status word: the tensor-core kernel's waits are bounded and write
 * RMLK_ERR_TIMEOUT there (instead of hanging) if a copy or MMA never completes.  NULL = not reported. */
RMLK_API int rmlk_b200_matmul_ex(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                        const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                        int64_t c_batch_stride, void* workspace, size_t workspace_bytes, int* status);
/* Same, with hints.  RMLK_MATMUL_B_STATIC: nothing still in flight on the device writes B (model weights).  The
 * kernels of this library let the next kernel of a stream be scheduled while the previous one drains, each waiting for
 * its predecessor before it touches memory; with this flag the tensor-core kernel requests its first tiles of B
 * before that wait, so the weight stream starts under the tail of the previous kernel.  flags = 0: as _ex. */
#define RMLK_MATMUL_B_STATIC 1
RMLK_API int rmlk_b200_matmul_flags(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                           const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                           int64_t c_batch_stride, void* workspace, size_t workspace_bytes, int* status, int flags);
/* C[:, 0:n] = A x B[:, 0:n] on a block of n columns: b and c point at the block's first column inside matrices whose rows
 * are ld elements apart.  A wide product (the logits of a language model, [64, 2048] x [2048, 128256]) can so be issued
 * block by block and each block copied to the host while the next is computed.  Only for shapes the tensor-core kernel
 * runs without a K split (rmlk_b200_matmul_window_supported); same kernel, same values as rmlk_b200_matmul_ex. */
RMLK_API int rmlk_b200_matmul_window(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, const void* b,
                            void* c, int64_t ld, int* status, int flags);
RMLK_API int rmlk_b200_matmul_window_supported(int64_t m, int64_t n, int64_t k, int64_t ld);
/* Unbatched MatMul for a caller that adds split-K partial sums in its own next kernel (rmlk_b200_add_rmsnorm does).
 * When the kernel plan for the shape splits K through the workspace, the [*parts][m*n] slabs are left in `workspace`
 * (to be added in slab order starting from 0.f - the order rmlk_b200_matmul uses) and c is NOT written; otherwise c
 * holds the result and *parts = 1.  Same kernels as rmlk_b200_matmul_ex (cuda/src/kernels/gemm.rs:206-231 in the
 * reference has no such form: cuBLAS reduces internally). */
RMLK_API int rmlk_b200_matmul_parts(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, int64_t k, const void* a, const void* b,
                           void* c, void* workspace, size_t workspace_bytes, int* status, int flags, int* parts);
/* dst[i] = 0.f + src[0][i] + ... + src[parts-1][i] (slabs of n floats, dense): the split-K reduction that
 * rmlk_b200_matmul runs after a workspace split, for callers of rmlk_b200_matmul_parts that need the plain result. */
RMLK_API int rmlk_b200_sum_parts(rmlk_stream_t stream, int dtype, int parts, int64_t n, const void* src, void* dst);
/* C[b] = A[b] x B[b]^T with B stored [n,k] row-major: what MatMul(A, Transpose(B, swap of the last two dims))
 * computes in the reference through a Transpose copy (cuda/src/kernels/transpose.rs:38-80) followed by
 * cublasGemmStridedBatchedEx (cuda/src/kernels/gemm.rs:206-231), without the copy.  A is [m,k], C is [m,n],
 * dense; batch strides in elements.  dtype f32. */
RMLK_API int rmlk_b200_matmul_nt(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                        const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                        int64_t c_batch_stride);
/* MatMul for callers that cannot allocate device memory and have no workspace to lend.  (No counterpart in
 * the reference: its cuBLAS handle allocates its own workspace, cuda/src/kernels/gemm.rs:119.)
 * Some hosts of this library run where cudaMalloc is off limits: inside a latency-critical serving loop,
 * where an allocation would stall every stream of the device; under a fixed memory budget that was carved up
 * at start-up; or from a plug-in that is only handed input and output buffers.  For them the split-K
 * scratch that rmlk_b200_matmul takes as `workspace` lives in a fixed array inside the library:
 * rmlk_b200_matmul_static_scratch_bytes() bytes (8 MiB) of device memory on every GPU that loads the
 * library, held until the process exits.  Same arguments and results as rmlk_b200_matmul_ex otherwise.
 *  - Shapes whose least scratch need exceeds the array are rejected with RMLK_ERR_INVALID_ARG; nothing is launched
 *    (rmlk_b200_matmul_static_supported answers beforehand).
 *  - The first call on each device looks up the array's device address and, like the first call of any
 *    MatMul here, configures the kernels it launches (cudaFuncSetAttribute, cudaGetDriverEntryPoint); make that
 *    first call outside any stream capture and before other threads call in.  No call allocates or frees
 *    device memory.
 *  - All calls share the one array and it keeps the previous call's partial sums; every call overwrites what
 *    it reads, so nothing needs clearing, but two calls that overlap on the GPU (different streams) race on
 *    it.  Keep calls on one stream, or order them with events. */
RMLK_API int rmlk_b200_matmul_static(rmlk_stream_t stream, int dtype, int64_t batch, int64_t m, int64_t n, int64_t k,
                            const void* a, int64_t a_batch_stride, const void* b, int64_t b_batch_stride, void* c,
                            int64_t c_batch_stride, int* status);
RMLK_API size_t rmlk_b200_matmul_static_scratch_bytes(void);
/* 1 if rmlk_b200_matmul_static takes the shape (its least scratch need fits the built-in array), 0 if it would be rejected. */
RMLK_API int rmlk_b200_matmul_static_supported(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k);
RMLK_API size_t rmlk_b200_matmul_workspace_bytes(int dtype, int64_t batch, int64_t m, int64_t n, int64_t k);

/* y[m, n] = alpha * y + beta * c, in place, c read through element strides (0 broadcasts a dimension; c = NULL: y = alpha * y).
 * The epilogue of ONNX Gemm after the MatMul: replaces the reference's alpha inside the cuBLAS call
 * (runtime/src/providers/cuda/backend/gemm.rs:181-191) and its add_alpha_beta_inplace kernel for the bias
 * (backend/gemm.rs:42-91, cuda/src/kernels/binary.rs compute_alpha_beta_inplace).  dtype f32 or f16 (arithmetic in fp32). */
RMLK_API int rmlk_b200_scale_add_bias(rmlk_stream_t stream, int dtype, int64_t m, int64_t n, void* y, float alpha, const void* c,
                             int64_t c_row_stride, int64_t c_col_stride, float beta);

/* ---- column-split MatMul across the GPUs of one NVLink domain ------------------------------------------------------
 * Y[m, n_total] = X[m, k] x W[k, n_total] with W split by columns over `world` ranks (one process per GPU).  The
 * reference has no multi-GPU path (runtime/src/core/plan.rs:4-28 is a placeholder); where it would gather shard results
 * with a collective after cublasGemmStridedBatchedEx (cuda/src/kernels/gemm.rs:206-231), this entry point has the rank
 * that computes a block of columns store it into EVERY rank's output buffer from the MatMul kernel's epilogue (ordinary
 * stores through peer mappings, over NVLink) and then raise a flag on every rank.
 *
 * Set-up (the caller's, once): every rank allocates an output buffer [m_max, n_total] floats and a flag array of
 * `world` 32-bit words (zero-filled), makes both reachable from the other ranks (CUDA IPC or a symmetric-memory
 * allocator) and fills rmlk_tp_peers with the addresses as seen from ITS OWN process: out[r] / flags[r] = rank r's
 * buffers, r = 0..world-1 (out[rank] / flags[rank] are the local ones).
 * A call: rmlk_b200_matmul_tp computes this rank's columns [col0, col0 + n_shard) from its shard w_shard[k, n_shard]
 * (dense) and a[m, k] (the same on every rank), stores them into all `world` outputs and sets word `rank` of every
 * flag array to `epoch`.  rmlk_b200_tp_wait then makes the stream wait until all words of the LOCAL flag array have
 * reached `epoch`: what follows on the stream sees the complete Y.  The wait is bounded (a second or two): if a rank
 * never arrives, RMLK_ERR_TIMEOUT is stored in *status (device word, may be NULL) and the stream goes on.
 * Epochs must grow by one per call (all ranks alike).  A rank may be a call ahead of another, so the caller alternates
 * between two output buffers (even / odd epochs); with that, stream order on every rank makes reuse safe.
 * dtype f32; n_shard, col0 and n_total multiples of 4.  `workspace`: rmlk_b200_matmul_tp_workspace_bytes() bytes. */
#define RMLK_TP_MAX_WORLD 8
typedef struct rmlk_tp_peers {
    int world, rank;
    void* out[RMLK_TP_MAX_WORLD];
    void* flags[RMLK_TP_MAX_WORLD];
} rmlk_tp_peers;
RMLK_API size_t rmlk_b200_matmul_tp_workspace_bytes(int dtype, int64_t m, int64_t n_shard, int64_t k);
RMLK_API int rmlk_b200_matmul_tp(rmlk_stream_t stream, int dtype, int64_t m, int64_t n_shard, int64_t k, const void* a, const void* w_shard,
                        int64_t n_total, int64_t col0, const rmlk_tp_peers* peers, unsigned int epoch, void* workspace,
                        size_t workspace_bytes, int* status);
RMLK_API int rmlk_b200_tp_wait(rmlk_stream_t stream, const void* local_flags, int world, unsigned int epoch, int* status);

/* ---- op chains as one launch ----------------------------------------------------------------------------------
 * The reference has no fused ops: an exported decoder graph reaches it as single ops, each dispatched to its own
 * backend (runtime/src/providers/cuda/backend/mod.rs:121-161).  The four entry points below compute exactly what
 * those chains compute (same fp32 expressions in the same order; the row sums may associate differently), f32 only.
 * The host runtime substitutes them when it recognises the chain; callers may also use them directly. */

/* RMSNorm as exported: Pow(x, exponent) -> ReduceMean(last axis, keepdims) -> Add(eps) -> Sqrt -> Div(x, .) -> Mul(., w).
 * x, out: [rows, cols] dense; weight: [cols].  Replaces one launch each of backend/pow.rs:123-132,
 * reduce_mean.rs:47-310, add.rs, sqrt.rs, div.rs, mul.rs. */
RMLK_API int rmlk_b200_rmsnorm(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* x, float exponent, float eps,
                      const void* weight, void* out);

/* Residual Add followed by RMSNorm: sum_out = a + b, norm_out = RMSNorm(sum_out) as above, one launch.  b may be the
 * b_parts >= 1 split-K slabs left by rmlk_b200_matmul_parts (slab stride b_part_stride elements), added in slab order
 * before the Add, so the values equal MatMul -> Add -> RMSNorm run op by op.  a, b slabs, sum_out, norm_out: [rows, cols]
 * dense; sum_out must not overlap a or b.  Replaces backend/add.rs plus the RMSNorm chain's launches. */
RMLK_API int rmlk_b200_add_rmsnorm(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* a, const void* b, int b_parts,
                          int64_t b_part_stride, float exponent, float eps, const void* weight, void* sum_out, void* norm_out);

/* Rotary embedding as exported: Add(Mul(x, cos), Mul(Concat(Neg(x[..., D/2:]), x[..., :D/2]), sin)).  shape4 = output dims
 * [d0, d1, d2, D] (dense output); *_strides = element strides of x / cos / sin per output dim, 0 to broadcast (x may be
 * a permuted view).  Replaces backend/mul.rs (x2), slice.rs:49-464 (x2), neg.rs, concat.rs:28-198, add.rs. */
RMLK_API int rmlk_b200_rope(rmlk_stream_t stream, int dtype, const int64_t* shape4, const int64_t* x_strides,
                   const int64_t* cos_strides, const int64_t* sin_strides, const void* x, const void* cosv, const void* sinv,
                   void* out);

/* Same, with the output placed by the caller: out_strides = element strides of the output per dim (NULL = dense).
 * Lets the rotated keys of a decode step be written straight into their slot of a carried KV cache instead of being
 * copied there by Concat (backend/concat.rs:28-198 re-copies the whole cache). */
RMLK_API int rmlk_b200_rope_to(rmlk_stream_t stream, int dtype, const int64_t* shape4, const int64_t* x_strides,
                      const int64_t* cos_strides, const int64_t* sin_strides, const void* x, const void* cosv, const void* sinv,
                      void* out, const int64_t* out_strides);

/* The additive attention mask of an exported decoder as one launch, out [batch, 1, s_len, t_len] f32:
 *   Where(Equal(Cast(attention_mask [batch, t_len] i64 -> f32), cmp_pad), v_pad,
 *         Where(Equal(Trilu(ConstantOfShape([s_len, t_len], fill), k, upper = 1), cmp_tri), v_future, v_else))
 * Replaces backend/constant_of_shape.rs, trilu.rs, equal.rs (x2), whereop.rs (x2), cast.rs: seven launches, same bits (only
 * comparisons and selections of the given constants). */
RMLK_API int rmlk_b200_causal_padding_mask(rmlk_stream_t stream, int64_t batch, int64_t s_len, int64_t t_len, int64_t k,
                                  const void* attention_mask, float fill, float cmp_tri, float v_future, float v_else,
                                  float cmp_pad, float v_pad, void* out);

/* The cos / sin tables of a rotary embedding as exported: f = Mul(a, b) with a [rows] (positions, one per row) and b [half]
 * (inverse frequencies), emb = Concat(f, f) on the last axis, cos_out = Cos(emb), sin_out = Sin(emb), both [rows, 2 half].
 * Replaces backend/mul.rs, concat.rs:28-198, cos.rs and sin.rs (four launches) with one; same functions, same bits. */
RMLK_API int rmlk_b200_rope_tables(rmlk_stream_t stream, int dtype, int64_t rows, int64_t half, const void* a, const void* b, void* cos_out,
                          void* sin_out);

/* Several small placements as ONE launch: rotary embeddings (as rmlk_b200_rope_to) and strided -> strided copies of 4-byte
 * elements (as rmlk_b200_strided_copy_to, rank <= 5), e.g. the rotated queries, the rotated keys into their cache slot and
 * the new values into theirs, which a decode step would otherwise issue as three launches of a few microseconds each.
 * The jobs must be independent of one another (no job reads what another writes).  Every job may read its input as the
 * sum of `in_parts` split-K slabs `in_part_stride` elements apart, added in slab order starting from 0.f as
 * rmlk_b200_sum_parts does (in_parts <= 1: a plain tensor).  At most RMLK_BATCH_MAX_JOBS jobs. */
#define RMLK_BATCH_MAX_JOBS 4
#define RMLK_BATCH_ROPE 0
#define RMLK_BATCH_COPY4 1
typedef struct rmlk_batch_job {
    int kind;                /* RMLK_BATCH_ROPE | RMLK_BATCH_COPY4 */
    int rank;                /* ROPE: 4; COPY4: 1..5 */
    int in_parts;            /* split-K slabs of the input (0 or 1: none) */
    int reserved;
    int64_t in_part_stride;  /* elements between slabs */
    int64_t shape[5];
    int64_t in_strides[5];   /* element strides */
    int64_t out_strides[5];
    int64_t cos_strides[4];  /* ROPE only */
    int64_t sin_strides[4];
    const void* in;
    const void* cosv;
    const void* sinv;
    void* out;
} rmlk_batch_job;
RMLK_API int rmlk_b200_rope_copy_batch(rmlk_stream_t stream, int n_jobs, const rmlk_batch_job* jobs);

/* Decode attention over a KV cache read in place, one launch: for each of `problems` (batch entry x KV head) and each
 * of its `rows` (1..4) query rows - the query heads sharing that KV head, one new token each -
 *   out[p][r] = softmax_t((q[p][r] . K[p][t]) * scale + mask[b][h][t]) . V[p][:, :]
 * q, out: [problems, rows, head_dim] dense; K, V: [keys, head_dim] dense rows per problem, problems
 * k_problem_stride / v_problem_stride elements apart (a cache with spare room); mask: rows of `keys` floats found at
 * b * mask_batch_stride + h * mask_head_stride with b = p / kv_heads, h = (p % kv_heads) * rows + r, or NULL.
 * head_dim 16 / 32 / 64 / 128, keys <= 12288 (rmlk_b200_gqa_decode_attention_supported).  Replaces, for a decode
 * step, backend/expand.rs (x2), transpose.rs, matmul.rs (x2), mul.rs, add.rs, softmax.rs - each a launch with its own
 * copy in the reference - and reads K and V once. */
RMLK_API int rmlk_b200_gqa_decode_attention(rmlk_stream_t stream, int dtype, int64_t problems, int64_t rows, int64_t head_dim, int64_t keys,
                                   int64_t kv_heads, const void* q, const void* k, int64_t k_problem_stride, const void* v,
                                   int64_t v_problem_stride, float scale, const void* mask, int64_t mask_batch_stride,
                                   int64_t mask_head_stride, void* out);
RMLK_API int rmlk_b200_gqa_decode_attention_supported(int64_t rows, int64_t head_dim, int64_t keys);
/* Same, with the keys of a problem split over several CTAs (128 keys each) when `workspace` holds at least
 * rmlk_b200_gqa_decode_attention_workspace_bytes(...) bytes: partial softmax results are merged through the workspace
 * by the CTA that finishes last for a problem.  The first 16 * problems bytes of the workspace (arrival counters)
 * must be zero on entry and are zero again on exit; the rest needs no initialisation.  Without a workspace, or for
 * 128 keys or fewer, the one-CTA-per-problem kernel above runs. */
RMLK_API int rmlk_b200_gqa_decode_attention_ws(rmlk_stream_t stream, int dtype, int64_t problems, int64_t rows, int64_t head_dim, int64_t keys,
                                      int64_t kv_heads, const void* q, const void* k, int64_t k_problem_stride, const void* v,
                                      int64_t v_problem_stride, float scale, const void* mask, int64_t mask_batch_stride,
                                      int64_t mask_head_stride, void* out, void* workspace, size_t workspace_bytes);
RMLK_API size_t rmlk_b200_gqa_decode_attention_workspace_bytes(int64_t problems, int64_t rows, int64_t head_dim, int64_t keys);

/* SwiGLU gate as exported: Mul(Mul(gate, Sigmoid(gate)), up), n elements each.  Replaces backend/sigmoid.rs (cuDNN
 * activation, kernels/activation.rs:6-39) and backend/mul.rs (x2). */
RMLK_API int rmlk_b200_swiglu(rmlk_stream_t stream, int dtype, int64_t n, const void* gate, const void* up, void* out);
/* Same with gate and up given as [rows, cols] blocks of wider matrices (row pitches in elements; e.g. the two halves of
 * one MatMul against the concatenated gate and up weights); out is dense [rows, cols].  cols, pitches: multiples of 4. */
RMLK_API int rmlk_b200_swiglu_pitched(rmlk_stream_t stream, int dtype, int64_t rows, int64_t cols, const void* gate,
                             int64_t gate_pitch, const void* up, int64_t up_pitch, void* out);

/* Attention probabilities as exported: Softmax(Add(Mul(scores, scale), mask), last axis).  scores / out: [d0, d1, d2, cols]
 * dense (lead3 = d0, d1, d2); mask rows are dense, mask_strides3 = its element strides over d0, d1, d2 (0 = broadcast);
 * cols <= 2048.  Replaces backend/mul.rs, add.rs and softmax.rs:31-158 (cudnnSoftmaxForward). */
RMLK_API int rmlk_b200_scale_mask_softmax(rmlk_stream_t stream, int dtype, const int64_t* lead3, int64_t cols,
                                 const int64_t* mask_strides3, float scale, const void* scores, const void* mask, void* out);

#ifdef __cplusplus
}
#endif
#endif /* RMLK_B200_H */
