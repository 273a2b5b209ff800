// Column-split MatMul across the GPUs of one NVLink domain: Y[M, N] = X[M, K] x W[K, N] with W split by columns.
// Rank r holds W[:, col0 : col0 + n_shard] and computes that block of columns of Y; every rank needs all of Y.
// Instead of an all-gather after the MatMul, the rank that computes a block stores it into EVERY rank's [M, N] output
// buffer (the peers' buffers are mapped into its address space; the stores are ordinary global stores that cross
// NVLink), then raises a flag in every rank's flag array.  A rank's output is complete when the flags of all ranks
// have reached the call's epoch (rmlk_b200_tp_wait: a bounded wait that reports RMLK_ERR_TIMEOUT instead of hanging).
//
// For shapes the tensor-core kernels take, the stores to the peers happen in the MatMul kernel's own epilogue, tile by
// tile, so the NVLink traffic runs under the rest of the product.  Other shapes compute the block into scratch and one
// copy kernel spreads it.  No TMA access touches another GPU's memory and nothing here uses multicast: loads are local,
// peer traffic is plain stores and the flag words.
//
// The reference has no multi-GPU path (runtime/src/core/plan.rs:4-28 is a placeholder).
#include "common.cuh"

namespace rmlk {

bool tc_matmul_eligible(int64_t m, int64_t n, int64_t k, const void* a, const void* w, const void* c);
int tc_matmul(cudaStream_t st, int64_t m, int64_t n, int64_t k, const float* a, const float* w, float* c, void* workspace,
              size_t workspace_bytes, int* status, int* ksplit_out, int flags, int64_t ld, const TcPeers* peers);

struct TpDests {
    int n;
    float* out[RMLK_TP_MAX_WORLD];
};
struct TpFlags {
    int n;
    unsigned int* flag[RMLK_TP_MAX_WORLD];  // the word of THIS rank in every rank's flag array
};

// dense [m, n] block -> columns of every destination (row pitch ldc), 16 bytes per thread and step
__global__ void __launch_bounds__(256) tp_spread_kernel(const float4* __restrict__ src, TpDests d, int64_t m, int64_t n4, int64_t ldc4) {
    dep_sync();
    const int64_t total = m * n4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t r = i / n4, c = i - r * n4;
        const float4 v = src[i];
        for (int q = 0; q < d.n; q++) reinterpret_cast<float4*>(d.out[q])[r * ldc4 + c] = v;
    }
}

// sum of the split-K slabs [parts][m][n] (in slab order, starting from 0.f, as the MatMul's own reduction does) -> every destination
__global__ void __launch_bounds__(256) tp_sum_spread_kernel(const float4* __restrict__ slabs, int parts, TpDests d, int64_t m, int64_t n4, int64_t ldc4) {
    dep_sync();
    const int64_t total = m * n4;
    for (int64_t i = static_cast<int64_t>(blockIdx.x) * 256 + threadIdx.x; i < total; i += static_cast<int64_t>(gridDim.x) * 256) {
        const int64_t r = i / n4, c = i - r * n4;
        float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int k = 0; k < parts; k++) {
            const float4 v = slabs[static_cast<int64_t>(k) * total + i];
            s.x += v.x; s.y += v.y; s.z += v.z; s.w += v.w;
        }
        for (int q = 0; q < d.n; q++) reinterpret_cast<float4*>(d.out[q])[r * ldc4 + c] = s;
    }
}

// Runs after the kernels that stored the block (stream order): everything they wrote, to this GPU and to the peers, is
// ordered before the flag words by the system-scope fence and release stores.
__global__ void tp_signal_kernel(TpFlags f, unsigned int epoch) {
    dep_sync();
    __threadfence_system();
    if (threadIdx.x < f.n) asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(f.flag[threadIdx.x]), "r"(epoch) : "memory");
}

constexpr unsigned int TP_SPIN_LIMIT = 1u << 22;  // x >= 200 ns: a second or two, then the wait gives up

__global__ void tp_wait_kernel(const unsigned int* __restrict__ flags, int world, unsigned int epoch, int* status) {
    dep_sync();
    if (threadIdx.x < world) {
        bool seen = false;
        for (unsigned int spin = 0; spin < TP_SPIN_LIMIT; spin++) {
            unsigned int v;
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(flags + threadIdx.x) : "memory");
            if (static_cast<int>(v - epoch) >= 0) {  // epochs only grow (wrap-around safe)
                seen = true;
                break;
            }
            __nanosleep(200);
        }
        if (!seen && status) atomicExch(status, RMLK_ERR_TIMEOUT);
    }
    __threadfence_system();
}

}  // namespace rmlk

using namespace rmlk;

extern "C" size_t rmlk_b200_matmul_tp_workspace_bytes(int dtype, int64_t m, int64_t n_shard, int64_t k) {
    if (dtype != RMLK_F32 || m <= 0 || n_shard <= 0 || k <= 0) return 0;
    // room for the dense block (shapes that are spread by the copy kernel) in front of the MatMul's own scratch
    const size_t block = (static_cast<size_t>(m) * n_shard * sizeof(float) + 255) & ~static_cast<size_t>(255);
    return block + rmlk_b200_matmul_workspace_bytes(dtype, 1, m, n_shard, k);
}

extern "C" int rmlk_b200_matmul_tp(rmlk_stream_t stream, int dtype, int64_t m, int64_t n_shard, int64_t k, const void* a, const void* w_shard,
                                   int64_t n_total, int64_t col0, const rmlk_tp_peers* peers, unsigned int epoch, void* workspace,
                                   size_t workspace_bytes, int* status) {
    if (dtype != RMLK_F32) return fail(RMLK_ERR_UNSUPPORTED_DTYPE, "unsupported data type for matmul_tp (f32 only)");
    if (!peers) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: NULL peers");
    const int world = peers->world, rank = peers->rank;
    if (world < 1 || world > RMLK_TP_MAX_WORLD || rank < 0 || rank >= world) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: bad world / rank");
    if (m <= 0 || n_shard <= 0 || k <= 0 || n_total <= 0) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: extents must be positive");
    if (col0 < 0 || col0 + n_shard > n_total) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: the block of columns lies outside the output");
    if (n_shard % 4 || col0 % 4 || n_total % 4) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: column extents must be multiples of 4");
    if (!a || !w_shard) return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: NULL operand");
    for (int r = 0; r < world; r++)
        if (!peers->out[r] || !peers->flags[r] || !aligned_to(peers->out[r], 16))
            return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: every rank needs a 16-byte aligned output buffer and a flag array");
    cudaStream_t st = as_stream(stream);
    float* local = static_cast<float*>(peers->out[rank]) + col0;
    TcPeers tp;
    tp.n_peer = 0;
    tp.ldc = n_total;
    for (int r = 0; r < world; r++)
        if (r != rank) tp.out[tp.n_peer++] = static_cast<float*>(peers->out[r]) + col0;
    if (tc_matmul_eligible(m, n_shard, k, a, w_shard, local)) {
        // the MatMul kernel's epilogue stores every tile to all destinations
        int ksplit = 1;
        if (int rc = tc_matmul(st, m, n_shard, k, static_cast<const float*>(a), static_cast<const float*>(w_shard), local, workspace, workspace_bytes,
                               status, &ksplit, RMLK_MATMUL_B_STATIC, 0, &tp))
            return rc;
        if (ksplit > 1) {
            // few tiles and a long K: the plan split K through the scratch; the sum of the slabs goes to every destination
            TpDests d;
            d.n = world;
            for (int r = 0; r < world; r++) d.out[r] = static_cast<float*>(peers->out[r]) + col0;
            const int64_t total = m * (n_shard / 4);
            launch_dep(tp_sum_spread_kernel, dim3(flat_grid(total, 256, 8)), dim3(256), 0, st, reinterpret_cast<const float4*>(workspace), ksplit, d, m,
                       n_shard / 4, n_total / 4);
            RMLK_CHECK_LAUNCH("tp_sum_spread_kernel");
        }
    } else {
        const size_t block = (static_cast<size_t>(m) * n_shard * sizeof(float) + 255) & ~static_cast<size_t>(255);
        if (!workspace || workspace_bytes < block || !aligned_to(workspace, 16))
            return fail(RMLK_ERR_INVALID_ARG, "matmul_tp: this shape needs rmlk_b200_matmul_tp_workspace_bytes() of scratch");
        float* dense = static_cast<float*>(workspace);
        if (int rc = rmlk_b200_matmul_flags(stream, dtype, 1, m, n_shard, k, a, 0, w_shard, 0, dense, 0, static_cast<char*>(workspace) + block,
                                            workspace_bytes - block, status, RMLK_MATMUL_B_STATIC))
            return rc;
        TpDests d;
        d.n = world;
        for (int r = 0; r < world; r++) d.out[r] = static_cast<float*>(peers->out[r]) + col0;
        const int64_t total = m * (n_shard / 4);
        launch_dep(tp_spread_kernel, dim3(flat_grid(total, 256, 8)), dim3(256), 0, st, reinterpret_cast<const float4*>(dense), d, m, n_shard / 4, n_total / 4);
        RMLK_CHECK_LAUNCH("tp_spread_kernel");
    }
    TpFlags f;
    f.n = world;
    for (int r = 0; r < world; r++) f.flag[r] = static_cast<unsigned int*>(peers->flags[r]) + rank;
    launch_dep(tp_signal_kernel, dim3(1), dim3(32), 0, st, f, epoch);
    RMLK_CHECK_LAUNCH("tp_signal_kernel");
    return RMLK_OK;
}

extern "C" int rmlk_b200_tp_wait(rmlk_stream_t stream, const void* local_flags, int world, unsigned int epoch, int* status) {
    if (!local_flags || world < 1 || world > RMLK_TP_MAX_WORLD) return fail(RMLK_ERR_INVALID_ARG, "tp_wait: bad flag array / world");
    launch_dep(tp_wait_kernel, dim3(1), dim3(32), 0, as_stream(stream), static_cast<const unsigned int*>(local_flags), world, epoch, status);
    RMLK_CHECK_LAUNCH("tp_wait_kernel");
    return RMLK_OK;
}
