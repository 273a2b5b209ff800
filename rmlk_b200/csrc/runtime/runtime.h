// Host runtime types: graph description, tensors, device arena, instance.
// Host side of the operator path; the reference counterparts are cited in include/rmlk_b200_runtime.h.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include <map>
#include <memory>
#include <stdexcept>
#include <string>
#include <unordered_map>
#include <vector>

#include "../../../include/rmlk_b200_runtime.h"

namespace rmlk {
namespace rt {

// Error carrying an rmlk_status; thrown inside the runtime, converted at the C ABI.
struct Error : std::runtime_error {
    int code;
    Error(int c, const std::string& m) : std::runtime_error(m), code(c) {}
};
[[noreturn]] inline void raise(int code, const std::string& msg) { throw Error(code, msg); }
std::string dtype_name(int dt);
[[noreturn]] void unsupported_dtype(int dt, const char* what);

struct Attr {
    enum Kind { INT, INTS, FLOAT, STRING, TENSOR } kind = INT;
    int64_t i = 0;
    std::vector<int64_t> ints;
    float f = 0.f;
    std::string s;
    int t_dtype = RMLK_UNDEFINED;
    std::vector<int64_t> t_dims;
    std::vector<uint8_t> t_data;
};

struct ValueDef {
    std::string name;
    int dtype = RMLK_UNDEFINED;
    std::vector<int64_t> dims;  // 0 = dynamic
    bool is_input = false, is_output = false, is_const = false;
    std::shared_ptr<std::vector<uint8_t>> data;  // initializer payload (host), shared between graph copies
    const void* device_data = nullptr;           // or: initializer already resident on the device
};

struct NodeDef {
    int op = RMLK_OP_NOOP;
    std::vector<int> inputs;   // value ids, -1 = omitted optional input
    std::vector<int> outputs;  // value ids
    std::map<std::string, Attr> attrs;
};

struct Graph {
    std::vector<ValueDef> values;
    std::unordered_map<std::string, int> by_name;
    std::vector<NodeDef> nodes;
    int add_value(const std::string& name, int dtype, int rank, const int64_t* dims);
    int find(const std::string& name) const;
};

// Small integer / float tensors (shapes, axes, slice bounds, Range scalars) carry a host mirror so
// that shape inference never waits on the GPU.  The reference reads these back with a synchronous
// D2H copy in every op that needs them (e.g. backend/expand.rs:152-153, backend/slice.rs:276-334).
constexpr int64_t HOST_MIRROR_MAX = 64;

struct Storage;

struct Tensor {
    int dtype = RMLK_UNDEFINED;
    std::vector<int64_t> shape;  // empty = scalar
    void* data = nullptr;        // device
    Storage* storage = nullptr;  // arena ownership (null: weights, inputs, carried buffers)
    bool present = false;
    // Deferred layout op.  When `lazy` is set, `data` is the base of another tensor's buffer (kept alive
    // through `storage`) and element i of this tensor, in row-major order over `shape`, is element i in
    // row-major order over `pshape`, found at the element offset sum_d index_d * pstride[d] (stride 0 =
    // broadcast).  Expand and Transpose produce such views; Reshape and Flatten regroup `shape` and leave
    // pshape / pstride alone.  A consumer that cannot read strides gets a dense copy on demand (one
    // strided-copy launch for the whole chain); MatMul reads the view directly when it amounts to a
    // transposed and / or batch-broadcast right operand.  The reference copies in every one of these ops
    // (backend/expand.rs:49-216, backend/transpose.rs:44-178, backend/reshape.rs:27-73).
    bool lazy = false;
    std::vector<int64_t> pshape, pstride;
    // > 1: a MatMul result still in `parts` split-K slabs ([parts][numel] floats at `data`, to be added in slab
    // order); only ever set on a value whose single reader is the residual Add in front of an RMSNorm chain, which
    // adds the slabs itself.  Any other access goes through Instance::settle_parts first.
    int parts = 0;
    bool mirror_valid = false;
    std::vector<int64_t> mi;  // integer / bool mirror
    std::vector<double> mf;   // float mirror
    int64_t numel() const {
        int64_t n = 1;
        for (int64_t d : shape) n *= d;
        return n;
    }
    bool is_scalar() const { return shape.empty(); }
    size_t nbytes() const;
};

// Device memory for intermediates: bump allocation over large blocks plus a size-keyed free list, so
// that a buffer released after its last consumer was enqueued (single stream: stream order makes
// the reuse safe) serves a later op of the same run.  Everything is handed back at the start of the
// next run.  Replaces the reference's 4 KiB CudaBump with per-tensor cuMemAlloc fallback
// (runtime/src/providers/cuda/allocator.rs:96-139).
struct Storage {
    void* ptr = nullptr;
    size_t size = 0;
    int refs = 0;
};

class Arena {
  public:
    explicit Arena(size_t block_bytes) : block_bytes_(block_bytes) {}
    ~Arena();
    Storage* alloc(size_t bytes);
    void release(Storage* s);  // drop one reference; at zero the buffer returns to the free list
    void reset();
    size_t peak() const { return peak_; }

  private:
    struct Block {
        char* base;
        size_t size, used;
    };
    void* bump(size_t bytes);
    std::vector<Block> blocks_;
    std::multimap<size_t, void*> free_;
    std::vector<std::unique_ptr<Storage>> live_;
    size_t block_bytes_, bumped_ = 0, peak_ = 0;
};

// A persistent device buffer that grows geometrically.
struct DeviceBuffer {
    void* ptr = nullptr;
    size_t cap = 0;
    void* ensure(size_t bytes);
    void release();
};

struct Binding {  // output value -> input value, double-buffered
    int out_id, in_id;
    DeviceBuffer buf[2];
    int cur = 0;  // buffer the NEXT run writes
    Tensor carried;  // what the next run reads as the input
    bool have = false;
    // Growing cache: the bound output is Concat(bound input, new rows) along `axis` (a KV cache append).  The data
    // then lives in ONE buffer with room for `cap` entries along that axis; a run writes only the new rows behind
    // the old ones and hands out a strided view (Tensor::lazy, row pitch = cap), so nothing of the old cache is
    // copied.  The reference's Concat re-copies the whole cache every step (backend/concat.rs:28-76).
    bool appendable = false;
    int axis = 0;
    int64_t cap = 0;
    DeviceBuffer store;
    int64_t reserved_run = -1, reserved_tp = -1;  // run (and old length) for which room for the new rows was made
};

// A chain of single-op nodes that one fused launch can stand for (RMSNorm, rotary embedding, SwiGLU gate,
// scale + mask + softmax).  Found once per instance by matching the graph; the members other than the last one
// (`root`) are skipped when their turn comes, and at the root either the fused kernel runs or - when the
// tensors of this run do not meet its conditions - the members run one by one, as if nothing had been matched.
// Member outputs other than the root's are used only inside the chain, so running them late changes nothing.
struct FusedGroup {
    enum Kind { RMSNORM = 1, ROPE, SWIGLU, SCALE_MASK_SOFTMAX, ATTENTION, ROPE_TABLES, MASK } kind;
    int root = -1;
    int sub = -1;  // ATTENTION: index of the scale + mask + softmax group inside it, tried on its own when the whole does not fit
    std::vector<int> members;  // node indices in execution order, root last
    int v[12] = {-1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1, -1};  // value ids by role (per kind, see ops.cpp)
};

// MatMul nodes that multiply the SAME left operand by constant [K, N_i] weights (q / k / v projections, gate / up
// projections) run as one MatMul against the weights laid side by side ([K, sum N_i], built once on the device);
// each node's output is a block of columns of the product, handed out as a strided view.  One launch streams the
// activations once and gives the weight-streaming kernel a wide N instead of several narrow ones.
struct MergedMatMul {
    std::vector<int> nodes;     // member node indices, in execution order
    std::vector<int64_t> n, col0;
    int a_value = -1;
    int64_t k = 0, n_total = 0;
    DeviceBuffer w;             // the concatenated weights
    bool ready = false;
    int64_t done_in_run = -1;   // run counter of the run in which the first member produced every output
};

// A graph output that every run delivers to (pinned) host memory without being asked: the copy is enqueued as soon
// as the value exists - for a wide MatMul (the logits) block of columns by block of columns on a second stream, so
// that most of the transfer overlaps the rest of the product.  The reference copies outputs after the run
// (get_outputs, runtime/src/core/instance.rs:58-82).
struct HostOutput {
    int value_id = -1;
    void* dst = nullptr;
    size_t nbytes = 0;
    int64_t delivered_run = -1;  // run whose value is (being) copied
};

struct Instance {
    Graph g;
    std::vector<HostOutput> host_outputs;
    cudaStream_t copy_stream = nullptr;
    std::vector<cudaEvent_t> copy_events;   // chunk i of a run: recorded on `stream`, awaited by `copy_stream`
    cudaEvent_t copies_done = nullptr;      // recorded on `copy_stream` behind the last copy of a run
    bool copies_pending = false;
    int host_output_of(int value_id) const {
        for (size_t i = 0; i < host_outputs.size(); i++)
            if (host_outputs[i].value_id == value_id) return static_cast<int>(i);
        return -1;
    }
    void deliver_host_outputs();  // end of run: whatever was not streamed out while it was produced
    void wait_host_outputs();
    std::vector<MergedMatMul> merged;
    std::vector<int> merged_of_node;  // per node: index into `merged`, or -1
    int64_t run_counter = 0;
    void find_merged_matmuls();
    bool run_merged_matmul(int node_index);
    std::vector<FusedGroup> groups;
    std::vector<int> group_of_node;  // per node: index into `groups`, or -1
    bool fusion = true;              // RMLK_B200_NO_FUSION=1 turns the substitution off
    void find_fusions();
    bool run_fused(const FusedGroup& fg);
    int64_t fused_runs = 0, fused_fallbacks = 0;
    int device = 0;
    cudaStream_t stream = nullptr;
    bool own_stream = false;
    std::vector<Tensor> values;
    std::vector<DeviceBuffer> input_bufs;  // per value id (only inputs use theirs)
    DeviceBuffer weights;
    std::unique_ptr<Arena> arena;
    DeviceBuffer status_word;   // device int for gather / scatter_nd diagnostics
    DeviceBuffer matmul_ws;     // split-K scratch
    DeviceBuffer attn_ws;       // partial results + arrival counters of the split-keys attention kernel (kept zeroed)
    size_t attn_ws_zeroed = 0;  // capacity that has been zero-filled
    int64_t attn_ws_problems = -1;  // problem count of the last run that used attn_ws (its counter prefix is clean for that count)
    DeviceBuffer parts_ws;      // split-K slabs that outlive their MatMul (Tensor::parts)
    int parts_owner = -1;       // value id whose slabs are in parts_ws, -1: free
    std::vector<uint8_t> parts_ok_value;  // per value id: MatMul output read only by a residual Add + RMSNorm chain
    // per value id: the Concat node that appends this value (its only reader) to its first input, or -1.  The
    // producer of such rows may write them straight into the cache slot (rotary embedding of the keys does).
    std::vector<int> append_consumer;
    bool inplace_append_to = true;  // RMLK_B200_NO_APPEND_TO=1: new rows are made dense first, then copied in
    // Scores MatMul, softmax chain and context MatMul of a decode step run as one kernel, one CTA per problem (measured on
    // 512 problems of 4 query rows over 523 keys, head size 64: 27 us against 39 us for the three kernels it replaces).
    // RMLK_B200_ATTENTION=0 keeps the three kernels; =split uses the kernel that splits a problem's keys over CTAs of
    // 128 keys and combines them through a workspace (slower on that shape).
    bool attention = true;
    bool attention_split = false;
    bool add_norm = true;       // RMLK_B200_NO_ADD_NORM=1: keep the residual Add (and the split-K sum) as launches of their own
    void settle_parts(int value_id);
    DeviceBuffer read_staging;  // dense copy of a strided output while it is read back
    std::vector<Binding> bindings;
    std::vector<Tensor> const_nodes;       // per node: the materialised `value` of a Constant op
    std::vector<int> last_use;             // per value id: index of the last node reading it (-1: never)
    std::vector<uint8_t> input_fed;        // per value id: fed for the coming run
    std::vector<uint8_t> persistent;       // per value id: initializer / Constant output / input (kept across runs)
    std::vector<int> binding_of_out;       // per value id: index into `bindings` if it is a carried output, else -1
    int64_t launches = 0, syncs = 0;
    // host-side tracing (RMLK_B200_HOST_PROFILE=1): time spent enqueuing each op kind, printed at destruction
    bool host_profile = false;
    std::map<int, std::pair<int64_t, double>> host_prof;  // op -> (nodes run, microseconds)
    bool status_dirty = false;

    ~Instance();
    // gives `t` (the tensor of value `value_id`, dtype/shape already set) device memory
    void alloc_output(int value_id, Tensor& t);
    void run();
    // host view of a small tensor: mirror if valid, else a synchronous D2H copy
    std::vector<int64_t> host_i64(const Tensor& t);
    std::vector<double> host_f64(const Tensor& t);
    // Small placements of a decode step (rotary embeddings with a placed output, 4-byte strided copies into a cache
    // slot) are not launched where they come up but collected; whatever else is enqueued next - any kernel, copy or
    // synchronisation goes through check_rc / check_cuda - launches the collected jobs first, as one kernel.  Stream
    // order is therefore exactly what it would be without collecting.  RMLK_B200_NO_BATCH=1: every job launches at once.
    // Nodes whose inputs are all initializers (or outputs of such nodes) give the same result in every run - the inverse
    // frequencies of the rotary embedding are five of them in an exported Llama.  Their outputs are kept from the first run
    // on (copied into buffers of their own) and the nodes are skipped afterwards.  RMLK_B200_NO_FOLD=1: recomputed every run.
    bool fold_constants = true;
    std::vector<uint8_t> foldable;                 // per node
    std::vector<uint8_t> folded_ready;             // per node: outputs are in folded_out
    std::vector<std::vector<Tensor>> folded_out;   // per node: its outputs as persistent tensors
    std::vector<std::unique_ptr<DeviceBuffer>> folded_store;
    void find_foldable();
    bool batch_jobs = true;
    std::vector<rmlk_batch_job> pending_jobs;
    void defer_job(const rmlk_batch_job& job);
    void flush_jobs();
    // A merged q|k|v product whose split-K slabs have not been added up: `y` is the dense buffer the outputs' views point
    // into (not written yet; one reference is held here), the slabs lie in the MatMul workspace.  Collected jobs that read
    // from `y` are pointed at the slabs instead and add them up themselves; when the next thing is enqueued and anything
    // else still refers to `y`, the slabs are summed into it first - otherwise the sum never runs.
    struct Unsummed {
        Storage* y = nullptr;
        const float* slabs = nullptr;
        int parts = 0;
        int64_t part_stride = 0;
    } unsummed;
    void resolve_unsummed();
    void run_node(const NodeDef& n);
    void release_value(int value_id);
    // replaces a deferred view by a dense copy in arena memory (no-op for a dense tensor)
    void materialize(Tensor& t);
    void check_status();
};

size_t dtype_size_of(int dt);

std::string status_word_message(int word);  // text for a non-zero device status word
void check_cuda_fn(cudaError_t e, const char* what);
void check_rc_fn(int rc);
// launches the collected jobs of the instance that is running on this thread, if there are any
void flush_deferred();
// Every call into the kernel library and every CUDA call of the runtime is wrapped in one of these two: the collected
// jobs go out before whatever the wrapped expression enqueues (the comma operator evaluates left to right).
#define check_rc(expr) (::rmlk::rt::flush_deferred(), ::rmlk::rt::check_rc_fn(expr))
#define check_cuda(expr, what) (::rmlk::rt::flush_deferred(), ::rmlk::rt::check_cuda_fn((expr), (what)))

}  // namespace rt
}  // namespace rmlk
