/*
 * rmlk_b200 host runtime — the op backends and the sequential executor that sit above the kernel
 * launchers of rmlk_b200.h, behind a C ABI.
 *
 * This mirrors, for the operator path only, the host side of the reference:
 *   - graph construction:  rmlk_schema::GraphBuilder (schema/src/builder.rs:122-226)
 *   - instance creation:   rmlk_runtime::Builder::from_graph(..).build() (runtime/src/core/instance.rs:136-221)
 *   - one forward pass:    ModelInstance::run (runtime/src/core/instance.rs:89-119): load inputs, walk
 *                          the op list in order calling each op's backend, expose the outputs
 *   - per-op backends:     runtime/src/providers/cuda/backend/<op>.rs — dtype dispatch, ONNX shape
 *                          inference, broadcast strides, output allocation, kernel call
 *
 * Differences that are the point of this build (none changes a result):
 *   - no per-op PTX module load, handle creation, device `info` upload or D2H read of small
 *     operands: shapes/strides travel as kernel parameters, and small integer tensors (shapes, axes,
 *     slice bounds, Range scalars) carry a host mirror so that shape inference never waits on the GPU;
 *   - intermediates come from one device arena that is reset per run; initializers are uploaded once;
 *   - Reshape / Unsqueeze / Flatten are zero-copy views; Gather / Concat / Range run as kernels;
 *   - an output may be bound to an input (rmlk_instance_bind) so that e.g. a KV cache stays on the
 *     device across runs instead of crossing PCIe twice per step.
 *
 * Ops are identified by rmlk_schema::Op's discriminants (schema/src/op.rs:11-51).
 * All functions return RMLK_OK (0) or an rmlk_status code; rmlk_b200_last_error() has the text.
 */
#ifndef RMLK_B200_RUNTIME_H
#define RMLK_B200_RUNTIME_H

#include "rmlk_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    RMLK_OP_NOOP = 0, RMLK_OP_ADD = 1, RMLK_OP_CAST = 2, RMLK_OP_CONCAT = 3, RMLK_OP_CONV = 4, RMLK_OP_CONST = 5,
    RMLK_OP_CONSTANT_OF_SHAPE = 6, RMLK_OP_DIV = 7, RMLK_OP_EXPAND = 8, RMLK_OP_EQUAL = 9, RMLK_OP_FLATTEN = 10,
    RMLK_OP_GATHER = 11, RMLK_OP_GEMM = 12, RMLK_OP_GLOBAL_AVERAGE_POOL = 13, RMLK_OP_MAX_POOL = 14, RMLK_OP_MUL = 15,
    RMLK_OP_MATMUL = 16, RMLK_OP_POW = 17, RMLK_OP_RANGE = 18, RMLK_OP_RELU = 19, RMLK_OP_REDUCE_MEAN = 20,
    RMLK_OP_RESHAPE = 21, RMLK_OP_SCATTER_ND = 22, RMLK_OP_SHAPE = 23, RMLK_OP_SIGMOID = 24, RMLK_OP_SLICE = 25,
    RMLK_OP_SOFTMAX = 26, RMLK_OP_SQRT = 27, RMLK_OP_SUB = 28, RMLK_OP_TRANSPOSE = 29, RMLK_OP_TRILU = 30,
    RMLK_OP_UNSQUEEZE = 31, RMLK_OP_WHERE = 32, RMLK_OP_CONSTANT = 33, RMLK_OP_GREATER = 34, RMLK_OP_NEG = 35,
    RMLK_OP_SIN = 36, RMLK_OP_COS = 37
} rmlk_op;

typedef struct rmlk_graph rmlk_graph;
typedef struct rmlk_instance rmlk_instance;

/* ---- graph construction (GraphBuilder, schema/src/builder.rs) ---- */
RMLK_API rmlk_graph* rmlk_graph_create(void);
RMLK_API void rmlk_graph_destroy(rmlk_graph* g);
/* A graph input; a dim of 0 is dynamic (schema/src/builder.rs:122-155). */
RMLK_API int rmlk_graph_input(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims);
/* An initializer with host data of prod(dims) elements (rank 0 = scalar). */
RMLK_API int rmlk_graph_constant(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims,
                                 const void* data, size_t nbytes);
/* An initializer that already lives in device memory (weights loaded by another component): used in
 * place, never copied or freed; it must stay valid for as long as any instance built from the graph. */
RMLK_API int rmlk_graph_constant_device(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims,
                                        const void* device_data);
/* An intermediate or output value. */
RMLK_API int rmlk_graph_value(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims);
/* Appends an op node; returns its index (>= 0) or a negative rmlk_status.  An empty input name ("")
 * marks an omitted optional input. */
RMLK_API int rmlk_graph_op(rmlk_graph* g, int op, int n_inputs, const char* const* inputs, int n_outputs,
                           const char* const* outputs);
RMLK_API int rmlk_graph_attr_int(rmlk_graph* g, int node, const char* name, int64_t value);
RMLK_API int rmlk_graph_attr_ints(rmlk_graph* g, int node, const char* name, int n, const int64_t* values);
RMLK_API int rmlk_graph_attr_float(rmlk_graph* g, int node, const char* name, float value);
RMLK_API int rmlk_graph_attr_string(rmlk_graph* g, int node, const char* name, const char* value);
RMLK_API int rmlk_graph_attr_tensor(rmlk_graph* g, int node, const char* name, int dtype, int rank,
                                    const int64_t* dims, const void* data, size_t nbytes);
RMLK_API int rmlk_graph_output(rmlk_graph* g, const char* name);

/* ---- instance (Builder::build + ModelInstance, runtime/src/core/instance.rs) ---- */
/* Creates the instance on `device`, uploads all initializers in one pass, and reserves an arena of
 * `arena_bytes` (0 = default) for intermediates.  `stream` is the cudaStream_t every kernel is
 * enqueued on (NULL = a stream owned by the instance).  The graph may be destroyed afterwards. */
RMLK_API rmlk_instance* rmlk_instance_create(const rmlk_graph* g, int device, rmlk_stream_t stream, size_t arena_bytes);
RMLK_API void rmlk_instance_destroy(rmlk_instance* inst);
/* Feeds an input for the next run.  on_device == 0: `data` is host memory and is copied H2D on the
 * instance's stream (ExecutionState::load_value, runtime/src/core/execution_state.rs:117-196);
 * on_device != 0: `data` is a device pointer that is used in place and must stay valid until the
 * run has finished. */
RMLK_API int rmlk_instance_set_input(rmlk_instance* inst, const char* name, int dtype, int rank, const int64_t* dims,
                                     const void* data, int on_device);
/* After each run, graph output `output` becomes the value of graph input `input` for the next run
 * without leaving the device (double-buffered; no copy).  Until the first run the input must be fed
 * with rmlk_instance_set_input. */
RMLK_API int rmlk_instance_bind(rmlk_instance* inst, const char* output, const char* input);
/* Executes the op list once, in order (the loop of runtime/src/core/instance.rs:100-112).  Asynchronous:
 * returns when everything is enqueued, unless an op needed a device value on the host. */
RMLK_API int rmlk_instance_run(rmlk_instance* inst);
RMLK_API int rmlk_instance_synchronize(rmlk_instance* inst);
/* How the runtime reports a non-zero device status word when it next waits for the device (synchronize, read,
 * wait_outputs): 0 -> RMLK_OK; RMLK_ERR_TIMEOUT (a bounded wait inside a MatMul kernel expired) -> RMLK_ERR_TIMEOUT;
 * any other value (1 = index out of range, 2 = offset past the end, from Gather / ScatterND:
 * ScatterNdError::KernelFailed { code }, runtime/src/providers/cuda/backend/scatter_nd.rs:198-203) ->
 * RMLK_ERR_KERNEL_STATUS.  Pure host function. */
RMLK_API int rmlk_runtime_status_to_error(int status_word);
/* Shape / dtype / device address of a graph output (or any named value) after a run.  *device_ptr is NULL for an
 * output kept as a strided view: a bound output that is Concat(bound input, new rows) - a KV cache - lives in a
 * buffer with spare room along the concat axis and is appended in place (rmlk_instance_bind); rmlk_instance_read
 * still returns it dense.  RMLK_B200_NO_INPLACE_APPEND=1 in the environment keeps such outputs dense (one copy of
 * the whole cache per run, as the reference's Concat does, backend/concat.rs:28-76). */
RMLK_API int rmlk_instance_value_info(rmlk_instance* inst, const char* name, int* dtype, int* rank, int64_t* dims,
                                      void** device_ptr);
/* Registers host memory (pinned, for the copies to be asynchronous) that every following run delivers graph output
 * `name` to, without a read call: the copy is enqueued as soon as the value exists, and for a wide MatMul - the logits
 * of a language model - block of columns by block of columns on a second stream, while the rest of the product is
 * still being computed.  rmlk_instance_wait_outputs returns when the data of the last run has arrived.  host_dst =
 * NULL unregisters.  (The reference copies every output after the run, get_outputs, runtime/src/core/instance.rs:58-82.) */
RMLK_API int rmlk_instance_stream_output(rmlk_instance* inst, const char* name, void* host_dst, size_t nbytes);
RMLK_API int rmlk_instance_wait_outputs(rmlk_instance* inst);
/* Copies a value to host memory and waits for it (get_outputs, runtime/src/core/instance.rs:58-82). */
RMLK_API int rmlk_instance_read(rmlk_instance* inst, const char* name, void* dst, size_t nbytes);
/* Number of kernels / async copies enqueued by the last run, and number of times it had to wait for
 * the device (0 when all small operands had host mirrors). */
RMLK_API int64_t rmlk_instance_last_launches(const rmlk_instance* inst);
RMLK_API int64_t rmlk_instance_last_syncs(const rmlk_instance* inst);
/* Op chains that run as one launch (RMSNorm, rotary embedding, SwiGLU gate, scale + mask + softmax; see
 * rmlk_b200_rmsnorm ... in rmlk_b200.h): chains recognised in the graph, and, since the instance was created, how
 * often a chain ran fused / fell back to its single ops because a run's tensors did not meet the fused kernel's
 * conditions.  The reference executes every node on its own (runtime/src/core/instance.rs:100-112).
 * RMLK_B200_NO_FUSION=1 in the environment turns the substitution off. */
RMLK_API int64_t rmlk_instance_fused_chains(const rmlk_instance* inst);
RMLK_API int64_t rmlk_instance_fused_runs(const rmlk_instance* inst);
RMLK_API int64_t rmlk_instance_fused_fallbacks(const rmlk_instance* inst);
/* High-water mark of the intermediate arena, in bytes. */
RMLK_API size_t rmlk_instance_arena_peak(const rmlk_instance* inst);

#ifdef __cplusplus
}
#endif
#endif /* RMLK_B200_RUNTIME_H */
