// Graph container, device memory, the sequential executor and the C ABI of include/rmlk_b200_runtime.h.
#include "runtime.h"

#include <algorithm>
#include <chrono>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include "../common.cuh"

namespace rmlk {
namespace rt {

std::string dtype_name(int dt) {
    switch (dt) {
        case RMLK_F16: return "Float16"; case RMLK_F32: return "Float"; case RMLK_F64: return "Double";
        case RMLK_I32: return "Int32"; case RMLK_I64: return "Int64"; case RMLK_U8: return "Uint8"; case RMLK_I8: return "Int8";
        case RMLK_U16: return "Uint16"; case RMLK_I16: return "Int16"; case RMLK_U32: return "Uint32"; case RMLK_U64: return "Uint64";
        case RMLK_STRING: return "String"; case RMLK_BOOL: return "Bool";
        default: return "Undefined";
    }
}

// Message prefix matches the reference's UnsupportedDataType (runtime/src/core/error.rs:4-10).
void unsupported_dtype(int dt, const char* what) {
    raise(RMLK_ERR_UNSUPPORTED_DTYPE, std::string("unsupported data type: ") + dtype_name(dt) + " (" + what + ")");
}

void check_cuda_fn(cudaError_t e, const char* what) {
    if (e != cudaSuccess) raise(RMLK_ERR_CUDA_BASE + static_cast<int>(e), std::string(what) + ": " + cudaGetErrorString(e));
}

void check_rc_fn(int rc) {
    if (rc != RMLK_OK) raise(rc, rmlk_b200_last_error());
}

// the instance whose run() is executing on this thread (jobs are only ever collected inside run())
static thread_local Instance* tl_running = nullptr;

void flush_deferred() {
    if (!tl_running) return;
    if (!tl_running->pending_jobs.empty()) tl_running->flush_jobs();
    if (tl_running->unsummed.y) tl_running->resolve_unsummed();
}

void Instance::flush_jobs() {
    if (pending_jobs.empty()) return;
    std::vector<rmlk_batch_job> jobs;
    jobs.swap(pending_jobs);  // empty before anything is enqueued: the launch below goes through no check_rc macro
    if (unsummed.y) {
        // jobs that read the unsummed product read its slabs (same layout, `part_stride` elements apart)
        const char* lo = static_cast<const char*>(unsummed.y->ptr);
        const char* hi = lo + unsummed.y->size;
        for (rmlk_batch_job& j : jobs) {
            const char* in = static_cast<const char*>(j.in);
            if (in >= lo && in < hi && j.in_parts <= 1) {
                j.in = reinterpret_cast<const char*>(unsummed.slabs) + (in - lo);
                j.in_parts = unsummed.parts;
                j.in_part_stride = unsummed.part_stride;
            }
        }
    }
    check_rc_fn(rmlk_b200_rope_copy_batch(reinterpret_cast<rmlk_stream_t>(stream), static_cast<int>(jobs.size()), jobs.data()));
    launches++;
}

void Instance::resolve_unsummed() {
    if (!unsummed.y) return;
    Unsummed u = unsummed;
    unsummed = Unsummed();  // cleared first: nothing below goes through the check_rc macro, but keep the state simple
    if (u.y->refs > 1) {
        // a view of the product is still alive and may be read by what comes next: add the slabs up now
        check_rc_fn(rmlk_b200_sum_parts(reinterpret_cast<rmlk_stream_t>(stream), RMLK_F32, u.parts, u.part_stride, u.slabs, u.y->ptr));
        launches++;
    }
    arena->release(u.y);
}

// the byte range [lo, hi) a job's tensor covers (elements of 4 bytes; strides may be 0 or negative)
static void job_span(const void* base, int rank, const int64_t* shape, const int64_t* strides, int parts, int64_t part_stride, const char*& lo,
                     const char*& hi) {
    int64_t mn = 0, mx = 0;
    for (int d = 0; d < rank; d++) {
        const int64_t ext = (shape[d] > 0 ? shape[d] - 1 : 0) * strides[d];
        if (ext < 0) mn += ext; else mx += ext;
    }
    if (parts > 1) mx += static_cast<int64_t>(parts - 1) * part_stride;
    lo = static_cast<const char*>(base) + mn * 4;
    hi = static_cast<const char*>(base) + (mx + 1) * 4;
}

void Instance::defer_job(const rmlk_batch_job& job) {
    if (!batch_jobs || tl_running != this) {
        check_rc_fn((flush_deferred(), rmlk_b200_rope_copy_batch(reinterpret_cast<rmlk_stream_t>(stream), 1, &job)));
        launches++;
        return;
    }
    // a job may not read or overwrite what a collected job writes, nor overwrite what one reads: launch those first
    const int rank = job.kind == RMLK_BATCH_ROPE ? 4 : job.rank;
    const char *ilo, *ihi, *olo, *ohi;
    job_span(job.in, rank, job.shape, job.in_strides, job.in_parts, job.in_part_stride, ilo, ihi);
    job_span(job.out, rank, job.shape, job.out_strides, 0, 0, olo, ohi);
    bool clash = pending_jobs.size() >= RMLK_BATCH_MAX_JOBS;
    for (const rmlk_batch_job& p : pending_jobs) {
        const int pr = p.kind == RMLK_BATCH_ROPE ? 4 : p.rank;
        const char *plo, *phi, *qlo, *qhi;
        job_span(p.in, pr, p.shape, p.in_strides, p.in_parts, p.in_part_stride, plo, phi);
        job_span(p.out, pr, p.shape, p.out_strides, 0, 0, qlo, qhi);
        if ((ilo < qhi && qlo < ihi) || (olo < qhi && qlo < ohi) || (olo < phi && plo < ohi)) clash = true;
    }
    if (clash) flush_jobs();
    pending_jobs.push_back(job);
}

size_t Tensor::nbytes() const { return static_cast<size_t>(numel()) * dtype_size_of(dtype); }

// ---- Graph ------------------------------------------------------------------------------------
int Graph::add_value(const std::string& name, int dtype, int rank, const int64_t* dims) {
    if (name.empty()) raise(RMLK_ERR_INVALID_ARG, "value name must not be empty");
    if (by_name.count(name)) raise(RMLK_ERR_INVALID_ARG, "duplicate value name `" + name + "`");
    if (rank < 0 || (rank > 0 && !dims)) raise(RMLK_ERR_INVALID_ARG, "bad dims for value `" + name + "`");
    ValueDef v;
    v.name = name;
    v.dtype = dtype;
    v.dims.assign(dims, dims + rank);
    values.push_back(std::move(v));
    by_name[name] = static_cast<int>(values.size()) - 1;
    return static_cast<int>(values.size()) - 1;
}

int Graph::find(const std::string& name) const {
    auto it = by_name.find(name);
    return it == by_name.end() ? -1 : it->second;
}

// ---- Arena ------------------------------------------------------------------------------------
static size_t round_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

Arena::~Arena() {
    for (Block& b : blocks_) cudaFree(b.base);
}

void* Arena::bump(size_t bytes) {
    for (Block& b : blocks_) {
        if (b.size - b.used >= bytes) {
            void* p = b.base + b.used;
            b.used += bytes;
            bumped_ += bytes;
            peak_ = std::max(peak_, bumped_);
            return p;
        }
    }
    Block nb;
    nb.size = std::max(block_bytes_, bytes);
    nb.used = bytes;
    void* p = nullptr;
    check_cuda(cudaMalloc(&p, nb.size), "arena cudaMalloc");
    nb.base = static_cast<char*>(p);
    blocks_.push_back(nb);
    bumped_ += bytes;
    peak_ = std::max(peak_, bumped_);
    return p;
}

Storage* Arena::alloc(size_t bytes) {
    const size_t sz = round_up(std::max<size_t>(bytes, 1), 512);
    void* p = nullptr;
    size_t got = sz;
    auto it = free_.lower_bound(sz);
    if (it != free_.end() && it->first <= sz + sz / 2) {  // reuse only reasonably tight fits
        p = it->second;
        got = it->first;
        free_.erase(it);
    } else {
        p = bump(sz);
    }
    live_.emplace_back(new Storage{p, got, 1});
    return live_.back().get();
}

void Arena::release(Storage* s) {
    if (!s || s->refs <= 0) return;
    if (--s->refs == 0) free_.emplace(s->size, s->ptr);
}

void Arena::reset() {
    free_.clear();
    live_.clear();
    bumped_ = 0;
    if (blocks_.size() > 1) {  // consolidate so that later runs bump inside one block
        size_t total = 0;
        for (Block& b : blocks_) {
            total += b.size;
            cudaFree(b.base);
        }
        blocks_.clear();
        Block nb;
        nb.size = total + total / 8;
        nb.used = 0;
        void* p = nullptr;
        check_cuda(cudaMalloc(&p, nb.size), "arena cudaMalloc");
        nb.base = static_cast<char*>(p);
        blocks_.push_back(nb);
    } else {
        for (Block& b : blocks_) b.used = 0;
    }
}

void* DeviceBuffer::ensure(size_t bytes) {
    if (bytes <= cap && ptr) return ptr;
    size_t want = std::max<size_t>(round_up(bytes, 256), 256);
    if (cap) want = std::max(want, cap + cap / 2);
    void* p = nullptr;
    check_cuda(cudaMalloc(&p, want), "cudaMalloc");
    if (ptr) cudaFree(ptr);
    ptr = p;
    cap = want;
    return ptr;
}

void DeviceBuffer::release() {
    if (ptr) cudaFree(ptr);
    ptr = nullptr;
    cap = 0;
}

// ---- host mirrors -----------------------------------------------------------------------------
static bool mirror_from_host(Tensor& t, const void* host) {
    const int64_t n = t.numel();
    t.mirror_valid = false;
    t.mi.clear();
    t.mf.clear();
    if (n > HOST_MIRROR_MAX || !host) return false;
    const uint8_t* p = static_cast<const uint8_t*>(host);
    switch (t.dtype) {
        case RMLK_F32: t.mf.resize(n); for (int64_t i = 0; i < n; i++) { float v; std::memcpy(&v, p + 4 * i, 4); t.mf[i] = v; } break;
        case RMLK_F64: t.mf.resize(n); for (int64_t i = 0; i < n; i++) { double v; std::memcpy(&v, p + 8 * i, 8); t.mf[i] = v; } break;
        case RMLK_I64: case RMLK_U64: t.mi.resize(n); std::memcpy(t.mi.data(), p, 8 * n); break;
        case RMLK_I32: t.mi.resize(n); for (int64_t i = 0; i < n; i++) { int32_t v; std::memcpy(&v, p + 4 * i, 4); t.mi[i] = v; } break;
        case RMLK_U32: t.mi.resize(n); for (int64_t i = 0; i < n; i++) { uint32_t v; std::memcpy(&v, p + 4 * i, 4); t.mi[i] = v; } break;
        case RMLK_I16: t.mi.resize(n); for (int64_t i = 0; i < n; i++) { int16_t v; std::memcpy(&v, p + 2 * i, 2); t.mi[i] = v; } break;
        case RMLK_U16: t.mi.resize(n); for (int64_t i = 0; i < n; i++) { uint16_t v; std::memcpy(&v, p + 2 * i, 2); t.mi[i] = v; } break;
        case RMLK_I8: t.mi.resize(n); for (int64_t i = 0; i < n; i++) t.mi[i] = static_cast<int8_t>(p[i]); break;
        case RMLK_U8: t.mi.resize(n); for (int64_t i = 0; i < n; i++) t.mi[i] = p[i]; break;
        case RMLK_BOOL: t.mi.resize(n); for (int64_t i = 0; i < n; i++) t.mi[i] = p[i] != 0; break;
        default: return false;
    }
    t.mirror_valid = true;
    return true;
}

std::vector<int64_t> Instance::host_i64(const Tensor& t) {
    if (t.mirror_valid) {
        if (!t.mf.empty()) {
            std::vector<int64_t> r(t.mf.size());
            for (size_t i = 0; i < r.size(); i++) r[i] = static_cast<int64_t>(t.mf[i]);
            return r;
        }
        return t.mi;
    }
    // No mirror: wait for the device, as the reference does for every small operand.
    std::vector<uint8_t> raw(t.nbytes());
    if (!raw.empty()) {
        check_cuda(cudaMemcpyAsync(raw.data(), t.data, raw.size(), cudaMemcpyDeviceToHost, stream), "D2H of a small operand");
        check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        syncs++;
    }
    Tensor tmp;
    tmp.dtype = t.dtype;
    tmp.shape = {t.numel()};
    std::vector<int64_t> r;
    const int64_t n = t.numel();
    const uint8_t* p = raw.data();
    r.resize(n);
    for (int64_t i = 0; i < n; i++) {
        switch (t.dtype) {
            case RMLK_I64: case RMLK_U64: std::memcpy(&r[i], p + 8 * i, 8); break;
            case RMLK_I32: { int32_t v; std::memcpy(&v, p + 4 * i, 4); r[i] = v; break; }
            case RMLK_U32: { uint32_t v; std::memcpy(&v, p + 4 * i, 4); r[i] = v; break; }
            case RMLK_F32: { float v; std::memcpy(&v, p + 4 * i, 4); r[i] = static_cast<int64_t>(v); break; }
            case RMLK_F64: { double v; std::memcpy(&v, p + 8 * i, 8); r[i] = static_cast<int64_t>(v); break; }
            case RMLK_BOOL: case RMLK_U8: r[i] = p[i]; break;
            case RMLK_I8: r[i] = static_cast<int8_t>(p[i]); break;
            default: unsupported_dtype(t.dtype, "host read of a small operand");
        }
    }
    return r;
}

std::vector<double> Instance::host_f64(const Tensor& t) {
    if (t.mirror_valid) {
        if (!t.mf.empty() || t.mi.empty()) return t.mf;
        std::vector<double> r(t.mi.size());
        for (size_t i = 0; i < r.size(); i++) r[i] = static_cast<double>(t.mi[i]);
        return r;
    }
    std::vector<uint8_t> raw(t.nbytes());
    if (!raw.empty()) {
        check_cuda(cudaMemcpyAsync(raw.data(), t.data, raw.size(), cudaMemcpyDeviceToHost, stream), "D2H of a small operand");
        check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
        syncs++;
    }
    const int64_t n = t.numel();
    std::vector<double> r(n);
    for (int64_t i = 0; i < n; i++) {
        if (t.dtype == RMLK_F32) { float v; std::memcpy(&v, raw.data() + 4 * i, 4); r[i] = v; }
        else if (t.dtype == RMLK_F64) { std::memcpy(&r[i], raw.data() + 8 * i, 8); }
        else unsupported_dtype(t.dtype, "host read of a small float operand");
    }
    return r;
}

// ---- Instance ---------------------------------------------------------------------------------
Instance::~Instance() {
    if (host_profile) {
        double total = 0;
        for (auto& kv : host_prof) total += kv.second.second;
        fprintf(stderr, "[rmlk_b200 host profile] %.1f us of host time in ops\n", total);
        for (auto& kv : host_prof)
            fprintf(stderr, "  op %3d: %8lld nodes %10.1f us %6.2f us/node\n", kv.first, static_cast<long long>(kv.second.first), kv.second.second,
                    kv.second.second / std::max<int64_t>(1, kv.second.first));
    }
    cudaSetDevice(device);
    if (stream) cudaStreamSynchronize(stream);
    arena.reset();
    weights.release();
    status_word.release();
    matmul_ws.release();
    parts_ws.release();
    attn_ws.release();
    read_staging.release();
    if (copy_stream) {
        cudaStreamSynchronize(copy_stream);
        cudaStreamDestroy(copy_stream);
    }
    for (cudaEvent_t e : copy_events) cudaEventDestroy(e);
    if (copies_done) cudaEventDestroy(copies_done);
    for (DeviceBuffer& b : input_bufs) b.release();
    for (MergedMatMul& m : merged) m.w.release();
    for (Binding& b : bindings) {
        b.buf[0].release();
        b.buf[1].release();
        b.store.release();
    }
    if (own_stream && stream) cudaStreamDestroy(stream);
}

void Instance::alloc_output(int value_id, Tensor& t) {
    const size_t bytes = t.nbytes();
    if (binding_of_out[value_id] >= 0) {
        Binding& b = bindings[binding_of_out[value_id]];
        t.data = b.buf[b.cur].ensure(std::max<size_t>(bytes, 16));
        t.storage = nullptr;
        return;
    }
    t.storage = arena->alloc(bytes);
    t.data = t.storage->ptr;
}

void Instance::release_value(int value_id) {
    Tensor& t = values[value_id];
    if (t.storage) {
        arena->release(t.storage);
        t.storage = nullptr;
    }
}

void Instance::materialize(Tensor& t) {
    if (!t.lazy) return;
    Storage* base_storage = t.storage;
    const void* base = t.data;
    t.storage = arena->alloc(t.nbytes());
    t.data = t.storage->ptr;
    if (t.numel() > 0) {
        check_rc(rmlk_b200_strided_copy(reinterpret_cast<rmlk_stream_t>(stream), static_cast<int>(dtype_size_of(t.dtype)),
                                        static_cast<int>(t.pshape.size()), t.pshape.data(), t.pstride.data(), base, t.data));
        launches++;
    }
    if (base_storage) arena->release(base_storage);
    t.lazy = false;
    t.pshape.clear();
    t.pstride.clear();
}

// Adds up the split-K slabs a MatMul left behind (Tensor::parts) into an ordinary dense tensor: the path taken when
// the value is read by anything but the fused Add + RMSNorm kernel (that chain falling back to single ops).
void Instance::settle_parts(int value_id) {
    Tensor& t = values[value_id];
    if (t.parts <= 1) return;
    const void* slabs = t.data;
    const int parts = t.parts;
    t.parts = 0;
    t.storage = nullptr;
    alloc_output(value_id, t);
    check_rc(rmlk_b200_sum_parts(reinterpret_cast<rmlk_stream_t>(stream), t.dtype, parts, t.numel(), slabs, t.data));
    launches++;
    if (parts_owner == value_id) parts_owner = -1;
}

void Instance::deliver_host_outputs() {
    for (HostOutput& h : host_outputs) {
        if (h.delivered_run == run_counter) continue;
        Tensor& t = values[h.value_id];
        if (!t.present) continue;
        if (t.nbytes() != h.nbytes) raise(RMLK_ERR_INVALID_ARG, "host output `" + g.values[h.value_id].name + "`: size mismatch");
        if (t.parts > 1) settle_parts(h.value_id);
        const void* src = t.data;
        if (t.lazy && h.nbytes) {
            // a strided view (a carried cache with spare room) stays as it is: gathered into a staging buffer for the copy
            void* tmp = read_staging.ensure(h.nbytes);
            check_rc(rmlk_b200_strided_copy(reinterpret_cast<rmlk_stream_t>(stream), static_cast<int>(dtype_size_of(t.dtype)),
                                            static_cast<int>(t.pshape.size()), t.pshape.data(), t.pstride.data(), t.data, tmp));
            src = tmp;
        }
        if (h.nbytes) check_cuda(cudaMemcpyAsync(h.dst, src, h.nbytes, cudaMemcpyDeviceToHost, stream), "host output D2H");
        h.delivered_run = run_counter;
    }
    if (copies_pending) check_cuda(cudaEventRecord(copies_done, copy_stream), "cudaEventRecord");
}

void Instance::wait_host_outputs() {
    check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    if (copy_stream) check_cuda(cudaStreamSynchronize(copy_stream), "cudaStreamSynchronize");
    check_status();
}

void Instance::check_status() {
    if (!status_dirty) return;
    int code = 0;
    check_cuda(cudaMemcpyAsync(&code, status_word.ptr, sizeof(int), cudaMemcpyDeviceToHost, stream), "status D2H");
    check_cuda(cudaStreamSynchronize(stream), "cudaStreamSynchronize");
    status_dirty = false;
    if (code != 0) {
        check_cuda(cudaMemsetAsync(status_word.ptr, 0, sizeof(int), stream), "status reset");
        raise(rmlk_runtime_status_to_error(code), status_word_message(code));
    }
}

// The one device status word is shared by Gather / ScatterND (1 = index out of range, 2 = offset past the end:
// ScatterNdError::KernelFailed { code } in the reference, backend/scatter_nd.rs:198-203) and by the MatMul kernels,
// which store RMLK_ERR_TIMEOUT there when one of their bounded waits expires.
std::string status_word_message(int word) {
    if (word == RMLK_ERR_TIMEOUT) return "kernel failed: a bounded wait inside a MatMul kernel expired (code " + std::to_string(word) + "); its output is incomplete";
    return "kernel failed: index out of range (code " + std::to_string(word) + ")";
}

void Instance::find_foldable() {
    foldable.assign(g.nodes.size(), 0);
    folded_ready.assign(g.nodes.size(), 0);
    folded_out.assign(g.nodes.size(), {});
    if (!fold_constants) return;
    std::vector<uint8_t> constant(g.values.size(), 0);
    for (size_t v = 0; v < g.values.size(); v++) constant[v] = g.values[v].is_const ? 1 : 0;
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const NodeDef& n = g.nodes[i];
        if (n.op == RMLK_OP_NOOP || n.op == RMLK_OP_CONST || n.op == RMLK_OP_CONSTANT) continue;
        if (!group_of_node.empty() && group_of_node[i] >= 0) continue;     // members of a fused chain run at its last node
        if (!merged_of_node.empty() && merged_of_node[i] >= 0) continue;
        bool all = false;
        for (int v : n.inputs) {
            if (v < 0) continue;
            all = true;
            if (!constant[v]) {
                all = false;
                break;
            }
        }
        if (!all) continue;
        bool plain = true;
        for (int v : n.outputs)
            if (v >= 0 && (g.values[v].is_output || g.values[v].is_input)) plain = false;
        if (!plain) continue;
        foldable[i] = 1;
        for (int v : n.outputs)
            if (v >= 0) constant[v] = 1;
    }
}

void Instance::run() {
    // jobs are collected only while this function runs; whatever is left goes out before the outputs are delivered,
    // and nothing stays collected if the run ends with an error
    struct Running {
        Instance* self;
        Instance* before;
        explicit Running(Instance* s) : self(s), before(tl_running) { tl_running = s; }
        ~Running() {
            self->pending_jobs.clear();
            self->unsummed = Unsummed();  // (after an error; the arena is reset by the next run)
            tl_running = before;
        }
    } running(this);
    pending_jobs.clear();
    check_cuda(cudaSetDevice(device), "cudaSetDevice");
    launches = 0;
    syncs = 0;
    run_counter++;
    // hand back last run's intermediates
    for (size_t i = 0; i < values.size(); i++) {
        if (persistent[i]) continue;
        values[i].present = false;
        values[i].storage = nullptr;
        values[i].data = nullptr;
        values[i].lazy = false;
        values[i].parts = 0;
    }
    parts_owner = -1;
    if (copies_pending) {
        // last run's block-wise copies read buffers that this run is about to hand out again
        check_cuda(cudaStreamWaitEvent(stream, copies_done, 0), "cudaStreamWaitEvent");
        copies_pending = false;
    }
    arena->reset();
    for (Binding& b : bindings) {
        if (b.have && !input_fed[b.in_id]) {
            values[b.in_id] = b.carried;
            input_fed[b.in_id] = 1;
        }
    }
    for (size_t i = 0; i < values.size(); i++)
        if (g.values[i].is_input && !input_fed[i]) raise(RMLK_ERR_INVALID_ARG, "graph input `" + g.values[i].name + "` was not fed");
    for (size_t i = 0; i < g.nodes.size(); i++) {
        const NodeDef& n = g.nodes[i];
        const int gi = group_of_node.empty() ? -1 : group_of_node[i];
        if (gi >= 0) {
            // member of a fused chain: everything happens when the chain's last node comes up
            const FusedGroup& fg = groups[gi];
            if (fg.root != static_cast<int>(i)) continue;
            try {
                if (run_fused(fg)) {
                    fused_runs++;
                } else if (fg.kind == FusedGroup::ATTENTION) {
                    // scores MatMul, then the scale + mask + softmax chain (as one launch if it fits), then the context MatMul
                    const FusedGroup& sm = groups[fg.sub];
                    run_node(g.nodes[fg.members.front()]);
                    if (run_fused(sm)) {
                        fused_runs++;
                    } else {
                        fused_fallbacks++;
                        for (int m : sm.members) run_node(g.nodes[m]);
                    }
                    run_node(g.nodes[fg.root]);
                } else {
                    fused_fallbacks++;
                    for (int m : fg.members) run_node(g.nodes[m]);
                }
            } catch (const Error& e) {
                throw Error(e.code, std::string(e.what()) + " [fused chain ending at node " + std::to_string(i) + "]");
            }
            for (int m : fg.members) {
                for (int v : g.nodes[m].inputs)
                    if (v >= 0 && last_use[v] == static_cast<int>(i) && !g.values[v].is_output) release_value(v);
                for (int v : g.nodes[m].outputs)
                    if (v >= 0 && last_use[v] < 0 && !g.values[v].is_output) release_value(v);
            }
            continue;
        }
        if (i < foldable.size() && foldable[i] && folded_ready[i]) {
            // computed by an earlier run from initializers only: hand out the kept tensors
            for (size_t k = 0; k < n.outputs.size(); k++)
                if (n.outputs[k] >= 0) values[n.outputs[k]] = folded_out[i][k];
            continue;
        }
        try {
            if (host_profile) {
                const auto t0 = std::chrono::steady_clock::now();
                run_node(n);
                auto& slot = host_prof[n.op];
                slot.first++;
                slot.second += std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t0).count();
            } else {
                run_node(n);
            }
        } catch (const Error& e) {
            throw Error(e.code, std::string(e.what()) + " [node " + std::to_string(i) + ", op " + std::to_string(n.op) + "]");
        }
        if (i < foldable.size() && foldable[i]) {
            // first run: keep the outputs in buffers of their own, with their host mirrors.  A node whose output is a view
            // (Transpose / Expand of an initializer: no launch anyway) is left alone, so that its readers see the same
            // kind of operand in every run.
            bool view = false;
            for (int v : n.outputs) view = view || (v >= 0 && (values[v].lazy || values[v].parts > 1));
            if (view) {
                foldable[i] = 0;
                goto folded;
            }
            folded_out[i].assign(n.outputs.size(), Tensor());
            for (size_t k = 0; k < n.outputs.size(); k++) {
                if (n.outputs[k] < 0) continue;
                Tensor& t = values[n.outputs[k]];
                Tensor kept = t;
                kept.storage = nullptr;
                kept.parts = 0;
                if (t.present && t.nbytes() > 0) {
                    folded_store.emplace_back(new DeviceBuffer());
                    void* dst = folded_store.back()->ensure(t.nbytes());
                    check_cuda(cudaMemcpyAsync(dst, t.data, t.nbytes(), cudaMemcpyDeviceToDevice, stream), "keeping a constant result");
                    kept.data = dst;
                }
                folded_out[i][k] = kept;
            }
            folded_ready[i] = 1;
        }
    folded:
        if (n.op == RMLK_OP_GATHER || n.op == RMLK_OP_SCATTER_ND) status_dirty = true;
        for (int v : n.inputs)
            if (v >= 0 && last_use[v] == static_cast<int>(i) && !g.values[v].is_output) release_value(v);
        for (int v : n.outputs)
            if (v >= 0 && last_use[v] < 0 && !g.values[v].is_output) release_value(v);
    }
    flush_jobs();
    resolve_unsummed();
    deliver_host_outputs();
    for (Binding& b : bindings) {
        b.carried = values[b.out_id];
        b.carried.storage = nullptr;
        b.have = b.carried.present;
        b.cur ^= 1;
    }
    // inputs must be fed again for the next run unless a binding carries them
    std::fill(input_fed.begin(), input_fed.end(), 0);
}

}  // namespace rt
}  // namespace rmlk

// ---------------------------------------------------------------------------------------------
// C ABI
// ---------------------------------------------------------------------------------------------
using namespace rmlk::rt;

struct rmlk_graph {
    Graph g;
};
struct rmlk_instance {
    Instance I;
};

#define RT_TRY try {
#define RT_CATCH                                                          \
    }                                                                     \
    catch (const Error& e) { return rmlk::fail(e.code, e.what()); }       \
    catch (const std::exception& e) { return rmlk::fail(RMLK_ERR_INTERNAL, e.what()); }

extern "C" int rmlk_runtime_status_to_error(int word) {
    if (word == 0) return RMLK_OK;
    return word == RMLK_ERR_TIMEOUT ? RMLK_ERR_TIMEOUT : RMLK_ERR_KERNEL_STATUS;
}

extern "C" rmlk_graph* rmlk_graph_create(void) { return new (std::nothrow) rmlk_graph(); }
extern "C" void rmlk_graph_destroy(rmlk_graph* g) { delete g; }

extern "C" int rmlk_graph_input(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims) {
    RT_TRY
    if (!g || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    const int id = g->g.add_value(name, dtype, rank, dims);
    g->g.values[id].is_input = true;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_constant(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims, const void* data, size_t nbytes) {
    RT_TRY
    if (!g || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    int64_t n = 1;
    for (int i = 0; i < rank; i++) n *= dims[i];
    if (static_cast<size_t>(n) * dtype_size_of(dtype) != nbytes || (nbytes && !data) || dtype_size_of(dtype) == 0)
        raise(RMLK_ERR_INVALID_ARG, std::string("constant `") + name + "`: byte count does not match dims and dtype");
    const int id = g->g.add_value(name, dtype, rank, dims);
    ValueDef& v = g->g.values[id];
    v.is_const = true;
    v.data = std::make_shared<std::vector<uint8_t>>(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + nbytes);
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_constant_device(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims, const void* device_data) {
    RT_TRY
    if (!g || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    if (dtype_size_of(dtype) == 0) raise(RMLK_ERR_INVALID_ARG, std::string("constant `") + name + "`: bad dtype");
    const int id = g->g.add_value(name, dtype, rank, dims);
    ValueDef& v = g->g.values[id];
    int64_t n = 1;
    for (int i = 0; i < rank; i++) n *= dims[i];
    if (n && !device_data) raise(RMLK_ERR_INVALID_ARG, std::string("constant `") + name + "`: NULL device pointer");
    v.is_const = true;
    v.device_data = device_data;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_value(rmlk_graph* g, const char* name, int dtype, int rank, const int64_t* dims) {
    RT_TRY
    if (!g || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    g->g.add_value(name, dtype, rank, dims);
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_op(rmlk_graph* g, int op, int n_inputs, const char* const* inputs, int n_outputs, const char* const* outputs) {
    try {
        if (!g || n_inputs < 0 || n_outputs < 0) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
        NodeDef n;
        n.op = op;
        for (int i = 0; i < n_inputs; i++) {
            if (!inputs[i] || !inputs[i][0]) {
                n.inputs.push_back(-1);
                continue;
            }
            const int id = g->g.find(inputs[i]);
            if (id < 0) raise(RMLK_ERR_INVALID_ARG, std::string("unknown value `") + inputs[i] + "`");
            n.inputs.push_back(id);
        }
        for (int i = 0; i < n_outputs; i++) {
            const int id = g->g.find(outputs[i] ? outputs[i] : "");
            if (id < 0) raise(RMLK_ERR_INVALID_ARG, std::string("unknown value `") + (outputs[i] ? outputs[i] : "") + "`");
            n.outputs.push_back(id);
        }
        g->g.nodes.push_back(std::move(n));
        return static_cast<int>(g->g.nodes.size()) - 1;
    } catch (const Error& e) {
        return -rmlk::fail(e.code, e.what());
    } catch (const std::exception& e) {
        return -rmlk::fail(RMLK_ERR_INTERNAL, e.what());
    }
}

static NodeDef& node_at(rmlk_graph* g, int node) {
    if (!g || node < 0 || node >= static_cast<int>(g->g.nodes.size())) raise(RMLK_ERR_INVALID_ARG, "bad node index");
    return g->g.nodes[node];
}

extern "C" int rmlk_graph_attr_int(rmlk_graph* g, int node, const char* name, int64_t value) {
    RT_TRY
    Attr a;
    a.kind = Attr::INT;
    a.i = value;
    node_at(g, node).attrs[name] = a;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_attr_ints(rmlk_graph* g, int node, const char* name, int n, const int64_t* values) {
    RT_TRY
    Attr a;
    a.kind = Attr::INTS;
    if (n > 0) a.ints.assign(values, values + n);
    node_at(g, node).attrs[name] = a;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_attr_float(rmlk_graph* g, int node, const char* name, float value) {
    RT_TRY
    Attr a;
    a.kind = Attr::FLOAT;
    a.f = value;
    node_at(g, node).attrs[name] = a;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_attr_string(rmlk_graph* g, int node, const char* name, const char* value) {
    RT_TRY
    Attr a;
    a.kind = Attr::STRING;
    a.s = value ? value : "";
    node_at(g, node).attrs[name] = a;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_attr_tensor(rmlk_graph* g, int node, const char* name, int dtype, int rank, const int64_t* dims,
                                      const void* data, size_t nbytes) {
    RT_TRY
    Attr a;
    a.kind = Attr::TENSOR;
    a.t_dtype = dtype;
    if (rank > 0) a.t_dims.assign(dims, dims + rank);
    int64_t n = 1;
    for (int i = 0; i < rank; i++) n *= dims[i];
    if (static_cast<size_t>(n) * dtype_size_of(dtype) != nbytes) raise(RMLK_ERR_INVALID_ARG, "attribute tensor: byte count does not match dims and dtype");
    if (nbytes) a.t_data.assign(static_cast<const uint8_t*>(data), static_cast<const uint8_t*>(data) + nbytes);
    node_at(g, node).attrs[name] = a;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_graph_output(rmlk_graph* g, const char* name) {
    RT_TRY
    if (!g || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    const int id = g->g.find(name);
    if (id < 0) raise(RMLK_ERR_INVALID_ARG, std::string("unknown value `") + name + "`");
    g->g.values[id].is_output = true;
    return RMLK_OK;
    RT_CATCH
}

extern "C" rmlk_instance* rmlk_instance_create(const rmlk_graph* g, int device, rmlk_stream_t stream, size_t arena_bytes) {
    rmlk_instance* h = nullptr;
    try {
        if (!g) raise(RMLK_ERR_INVALID_ARG, "NULL graph");
        check_cuda(cudaSetDevice(device), "cudaSetDevice");
        h = new rmlk_instance();
        if (const char* e = getenv("RMLK_B200_HOST_PROFILE")) h->I.host_profile = e[0] == '1';
        Instance& I = h->I;
        I.g = g->g;
        I.device = device;
        if (stream) {
            I.stream = reinterpret_cast<cudaStream_t>(stream);
        } else {
            check_cuda(cudaStreamCreateWithFlags(&I.stream, cudaStreamNonBlocking), "cudaStreamCreate");
            I.own_stream = true;
        }
        I.arena.reset(new Arena(arena_bytes ? arena_bytes : (size_t(256) << 20)));
        const size_t nv = I.g.values.size();
        I.values.assign(nv, Tensor());
        I.input_bufs.resize(nv);
        I.input_fed.assign(nv, 0);
        I.last_use.assign(nv, -1);
        I.persistent.assign(nv, 0);
        I.binding_of_out.assign(nv, -1);
        for (size_t i = 0; i < nv; i++) I.persistent[i] = (I.g.values[i].is_const || I.g.values[i].is_input) ? 1 : 0;
        for (const NodeDef& n : I.g.nodes)
            if (n.op == RMLK_OP_CONSTANT && !n.outputs.empty()) I.persistent[n.outputs[0]] = 1;
        for (size_t i = 0; i < I.g.nodes.size(); i++)
            for (int v : I.g.nodes[i].inputs)
                if (v >= 0) I.last_use[v] = static_cast<int>(i);
        if (const char* e = getenv("RMLK_B200_NO_FUSION")) I.fusion = e[0] != '1';
        if (const char* e = getenv("RMLK_B200_NO_ADD_NORM")) I.add_norm = e[0] != '1';
        if (const char* e = getenv("RMLK_B200_NO_APPEND_TO")) I.inplace_append_to = e[0] != '1';
        if (const char* e = getenv("RMLK_B200_NO_BATCH")) I.batch_jobs = e[0] != '1';
        if (const char* e = getenv("RMLK_B200_NO_FOLD")) I.fold_constants = e[0] != '1';
        if (const char* e = getenv("RMLK_B200_ATTENTION")) {
            I.attention = e[0] != '0';
            I.attention_split = e[0] == 's';
        }
        I.find_fusions();  // recognise RMSNorm / rotary / SwiGLU / scale-mask-softmax chains; re-derives last_use
        I.find_merged_matmuls();  // q / k / v and gate / up projections: one MatMul per shared left operand
        I.find_foldable();        // nodes that depend on initializers only: computed in the first run, kept afterwards
        // one weight arena, one pass of uploads (the reference allocates and copies per tensor through a
        // 4 KiB bump allocator, runtime/src/providers/cuda/store.rs:95-262)
        size_t total = 0;
        std::vector<size_t> offs(nv, 0), node_off(I.g.nodes.size(), 0);
        for (size_t i = 0; i < nv; i++)
            if (I.g.values[i].is_const && !I.g.values[i].device_data) {
                offs[i] = total;
                total += round_up(std::max<size_t>(I.g.values[i].data ? I.g.values[i].data->size() : 0, 1), 256);
            }
        for (size_t k = 0; k < I.g.nodes.size(); k++) {
            const NodeDef& n = I.g.nodes[k];
            if (n.op != RMLK_OP_CONSTANT) continue;
            auto it = n.attrs.find("value");
            if (it == n.attrs.end() || it->second.kind != Attr::TENSOR) raise(RMLK_ERR_INVALID_ARG, "Constant op needs a tensor `value` attribute");
            node_off[k] = total;
            total += round_up(std::max<size_t>(it->second.t_data.size(), 1), 256);
        }
        char* base = static_cast<char*>(I.weights.ensure(std::max<size_t>(total, 256)));
        for (size_t i = 0; i < nv; i++) {
            const ValueDef& d = I.g.values[i];
            if (!d.is_const) continue;
            Tensor& t = I.values[i];
            t.dtype = d.dtype;
            t.shape = d.dims;
            t.present = true;
            if (d.device_data) {
                t.data = const_cast<void*>(d.device_data);
                continue;
            }
            t.data = base + offs[i];
            const size_t nb = d.data ? d.data->size() : 0;
            if (nb) check_cuda(cudaMemcpyAsync(t.data, d.data->data(), nb, cudaMemcpyHostToDevice, I.stream), "initializer upload");
            mirror_from_host(t, nb ? d.data->data() : nullptr);
        }
        for (size_t k = 0; k < I.g.nodes.size(); k++) {
            const NodeDef& n = I.g.nodes[k];
            if (n.op != RMLK_OP_CONSTANT) continue;
            const Attr& a = n.attrs.at("value");
            if (n.outputs.empty()) raise(RMLK_ERR_INVALID_ARG, "Constant op needs an output");
            Tensor& t = I.values[n.outputs[0]];
            t.dtype = a.t_dtype;
            t.shape = a.t_dims;
            t.data = base + node_off[k];
            t.present = true;
            if (!a.t_data.empty()) check_cuda(cudaMemcpyAsync(t.data, a.t_data.data(), a.t_data.size(), cudaMemcpyHostToDevice, I.stream), "constant upload");
            mirror_from_host(t, a.t_data.empty() ? nullptr : a.t_data.data());
        }
        I.status_word.ensure(256);
        check_cuda(cudaMemsetAsync(I.status_word.ptr, 0, 256, I.stream), "status init");
        check_cuda(cudaStreamSynchronize(I.stream), "cudaStreamSynchronize");
        // the host copies of the initializers are no longer needed by this instance
        for (ValueDef& d : I.g.values) d.data.reset();
        return h;
    } catch (const Error& e) {
        rmlk::fail(e.code, e.what());
    } catch (const std::exception& e) {
        rmlk::fail(RMLK_ERR_INTERNAL, e.what());
    }
    delete h;
    return nullptr;
}

extern "C" void rmlk_instance_destroy(rmlk_instance* inst) { delete inst; }

extern "C" int rmlk_instance_set_input(rmlk_instance* inst, const char* name, int dtype, int rank, const int64_t* dims, const void* data,
                                       int on_device) {
    RT_TRY
    if (!inst || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    Instance& I = inst->I;
    const int id = I.g.find(name);
    if (id < 0 || !I.g.values[id].is_input) raise(RMLK_ERR_INVALID_ARG, std::string("`") + name + "` is not a graph input");
    const ValueDef& d = I.g.values[id];
    if (dtype != d.dtype) raise(RMLK_ERR_INVALID_ARG, std::string("input `") + name + "`: dtype mismatch, expected " + dtype_name(d.dtype) + ", got " + dtype_name(dtype));
    // compare_shapes (runtime/src/utils/mod.rs:19-39): rank must match; a declared dim of 0 is dynamic
    if (rank != static_cast<int>(d.dims.size())) raise(RMLK_ERR_INVALID_ARG, std::string("input `") + name + "`: rank mismatch");
    for (int i = 0; i < rank; i++)
        if (d.dims[i] != 0 && d.dims[i] != dims[i]) raise(RMLK_ERR_INVALID_ARG, std::string("input `") + name + "`: dimensions mismatch");
    check_cuda(cudaSetDevice(I.device), "cudaSetDevice");
    Tensor& t = I.values[id];
    t = Tensor();
    t.dtype = dtype;
    t.shape.assign(dims, dims + rank);
    const size_t nb = t.nbytes();
    if (nb && !data) raise(RMLK_ERR_INVALID_ARG, std::string("input `") + name + "`: NULL data");
    if (on_device) {
        t.data = const_cast<void*>(data);
    } else {
        t.data = I.input_bufs[id].ensure(std::max<size_t>(nb, 16));
        if (nb) check_cuda(cudaMemcpyAsync(t.data, data, nb, cudaMemcpyHostToDevice, I.stream), "input upload");
        mirror_from_host(t, data);
    }
    t.present = true;
    I.input_fed[id] = 1;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_bind(rmlk_instance* inst, const char* output, const char* input) {
    RT_TRY
    if (!inst || !output || !input) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    Instance& I = inst->I;
    const int o = I.g.find(output), i = I.g.find(input);
    if (o < 0 || !I.g.values[o].is_output) raise(RMLK_ERR_INVALID_ARG, std::string("`") + output + "` is not a graph output");
    if (i < 0 || !I.g.values[i].is_input) raise(RMLK_ERR_INVALID_ARG, std::string("`") + input + "` is not a graph input");
    for (const Binding& b : I.bindings)
        if (b.out_id == o || b.in_id == i) raise(RMLK_ERR_INVALID_ARG, "value is already bound");
    Binding b;
    b.out_id = o;
    b.in_id = i;
    // output = Concat(input, something) along a fixed axis: a growing cache that can be appended in place
    if (!getenv("RMLK_B200_NO_INPLACE_APPEND"))
        for (const NodeDef& n : I.g.nodes) {
            if (n.outputs.empty() || n.outputs[0] != o) continue;
            auto ax = n.attrs.find("axis");
            if (n.op == RMLK_OP_CONCAT && n.inputs.size() == 2 && n.inputs[0] == i && n.inputs[1] >= 0 && ax != n.attrs.end() &&
                ax->second.kind == Attr::INT) {
                b.appendable = true;
                b.axis = static_cast<int>(ax->second.i);
            }
        }
    I.bindings.push_back(b);
    I.binding_of_out[o] = static_cast<int>(I.bindings.size()) - 1;
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_run(rmlk_instance* inst) {
    RT_TRY
    if (!inst) raise(RMLK_ERR_INVALID_ARG, "NULL instance");
    inst->I.run();
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_synchronize(rmlk_instance* inst) {
    RT_TRY
    if (!inst) raise(RMLK_ERR_INVALID_ARG, "NULL instance");
    check_cuda(cudaStreamSynchronize(inst->I.stream), "cudaStreamSynchronize");
    inst->I.check_status();
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_value_info(rmlk_instance* inst, const char* name, int* dtype, int* rank, int64_t* dims, void** device_ptr) {
    RT_TRY
    if (!inst || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    Instance& I = inst->I;
    const int id = I.g.find(name);
    if (id < 0) raise(RMLK_ERR_INVALID_ARG, std::string("unknown value `") + name + "`");
    const Tensor& t = I.values[id];
    if (!t.present) raise(RMLK_ERR_INVALID_ARG, std::string("value `") + name + "` has no data");
    if (dtype) *dtype = t.dtype;
    if (rank) *rank = static_cast<int>(t.shape.size());
    if (dims)
        for (size_t i = 0; i < t.shape.size() && i < RMLK_MAX_RANK; i++) dims[i] = t.shape[i];
    if (device_ptr) *device_ptr = t.lazy ? nullptr : t.data;  // a strided view (growing cache) has no dense buffer to hand out
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_read(rmlk_instance* inst, const char* name, void* dst, size_t nbytes) {
    RT_TRY
    if (!inst || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    Instance& I = inst->I;
    const int id = I.g.find(name);
    if (id < 0) raise(RMLK_ERR_INVALID_ARG, std::string("unknown value `") + name + "`");
    const Tensor& t = I.values[id];
    if (!t.present) raise(RMLK_ERR_INVALID_ARG, std::string("value `") + name + "` has no data");
    if (nbytes != t.nbytes()) raise(RMLK_ERR_INVALID_ARG, std::string("read of `") + name + "`: size mismatch");
    const void* src = t.data;
    if (t.lazy && nbytes) {
        // a strided view (a cache kept in a buffer with spare room): gather it into a dense staging buffer first
        void* tmp = I.read_staging.ensure(nbytes);
        check_rc(rmlk_b200_strided_copy(reinterpret_cast<rmlk_stream_t>(I.stream), static_cast<int>(dtype_size_of(t.dtype)),
                                        static_cast<int>(t.pshape.size()), t.pshape.data(), t.pstride.data(), t.data, tmp));
        src = tmp;
    }
    if (nbytes) check_cuda(cudaMemcpyAsync(dst, src, nbytes, cudaMemcpyDeviceToHost, I.stream), "output D2H");
    check_cuda(cudaStreamSynchronize(I.stream), "cudaStreamSynchronize");
    I.check_status();
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_stream_output(rmlk_instance* inst, const char* name, void* host_dst, size_t nbytes) {
    RT_TRY
    if (!inst || !name) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    Instance& I = inst->I;
    const int id = I.g.find(name);
    if (id < 0 || !I.g.values[id].is_output) raise(RMLK_ERR_INVALID_ARG, std::string("`") + name + "` is not a graph output");
    check_cuda(cudaSetDevice(I.device), "cudaSetDevice");
    I.wait_host_outputs();
    const int at = I.host_output_of(id);
    if (!host_dst) {
        if (at >= 0) I.host_outputs.erase(I.host_outputs.begin() + at);
        return RMLK_OK;
    }
    HostOutput h;
    h.value_id = id;
    h.dst = host_dst;
    h.nbytes = nbytes;
    if (at >= 0) I.host_outputs[at] = h;
    else I.host_outputs.push_back(h);
    if (!I.copy_stream) {
        check_cuda(cudaStreamCreateWithFlags(&I.copy_stream, cudaStreamNonBlocking), "cudaStreamCreate");
        check_cuda(cudaEventCreateWithFlags(&I.copies_done, cudaEventDisableTiming), "cudaEventCreate");
    }
    return RMLK_OK;
    RT_CATCH
}

extern "C" int rmlk_instance_wait_outputs(rmlk_instance* inst) {
    RT_TRY
    if (!inst) raise(RMLK_ERR_INVALID_ARG, "NULL argument");
    check_cuda(cudaSetDevice(inst->I.device), "cudaSetDevice");
    inst->I.wait_host_outputs();
    return RMLK_OK;
    RT_CATCH
}

extern "C" int64_t rmlk_instance_last_launches(const rmlk_instance* inst) { return inst ? inst->I.launches : 0; }
extern "C" int64_t rmlk_instance_last_syncs(const rmlk_instance* inst) { return inst ? inst->I.syncs : 0; }
extern "C" int64_t rmlk_instance_fused_chains(const rmlk_instance* inst) {
    if (!inst) return 0;
    int64_t n = 0;  // groups that own their nodes (a softmax chain inside an attention group is not counted twice)
    for (size_t i = 0; i < inst->I.groups.size(); i++) {
        const int root = inst->I.groups[i].root;
        if (root >= 0 && inst->I.group_of_node[root] == static_cast<int>(i)) n++;
    }
    return n;
}
extern "C" int64_t rmlk_instance_fused_runs(const rmlk_instance* inst) { return inst ? inst->I.fused_runs : 0; }
extern "C" int64_t rmlk_instance_fused_fallbacks(const rmlk_instance* inst) { return inst ? inst->I.fused_fallbacks : 0; }
extern "C" size_t rmlk_instance_arena_peak(const rmlk_instance* inst) { return inst && inst->I.arena ? inst->I.arena->peak() : 0; }
