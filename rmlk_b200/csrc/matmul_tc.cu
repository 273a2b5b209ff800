// fp32 MatMul on the 5th-generation tensor cores: tcgen05.mma kind::tf32 with a 3xTF32 split, operands
// brought in by TMA, accumulators and the weight operand in TMEM.  C[M,N] = A[M,K] x W[K,N], row-major fp32.
//
// Orientation.  W is the large, streamed operand.  One CTA owns 128 columns of W — the MMA's M dimension,
// one TMEM lane per column — and a tile of MT <= 128 rows of the activations A, the MMA's N dimension.
// The accumulator D[n][m] is 128 lanes x MT fp32 columns of TMEM, i.e. C transposed; the epilogue writes
// C[m][n0 + lane], coalesced across the lanes of a warp.
//
// 3xTF32.  x = hi + lo with hi = x truncated to tf32 (sign, exponent, 10 mantissa bits) and lo = x - hi, which
// is exact in fp32.  The MMA itself reads only the tf32 part of an operand word, so the raw fp32 word serves
// as hi without any conversion and only lo has to be computed (one AND, one subtraction).  Per k-step three
// MMAs' worth of products, hi*hi + hi*lo + lo*hi, accumulate in fp32 (the dropped lo*lo term is below 2^-20
// relative).  Two of them are issued as one MMA: an activation stage holds the lo tile followed by the raw tile, and a
// single descriptor with N = 2 MT covers both, so W_hi x [x_lo; x_hi] fills two accumulator blocks (an MMA costs about the
// same whatever its N; the number of MMAs per k-block is what bounds this kernel at small M).  W_lo x x_hi goes into the
// hi x lo block: the tensor core truncates when it adds into its accumulator, and keeping both small products out of
// the large hi x hi sums halves the error (about 5e-6 of the result's scale at K = 2048).  The epilogue adds the blocks.
//
// Data path per k-block of 32:
//   warp 0     TMA: one unswizzled [32 k][128 n] box of W (512-byte row pieces; four 32-wide boxes streamed a fifth
//              slower) into a ring of SW blocks
//   warp 10    TMA: one 128B-swizzled [MT][32 k] box of A into a ring of SA blocks
//   warps 2-9  converters (two groups of four warps on alternate k-blocks): thread (sub, lane) owns weight
//              column sub*32+lane: it reads its 32 k values from shared memory (conflict-free), and writes the
//              raw words and their lo parts straight into TMEM with tcgen05.st, so the weights never make a
//              second trip through shared memory - and the W block is handed back to the TMA right then, long
//              before the MMAs that use it complete; the lo part of the small A tile goes into a twin tile at
//              the same swizzled offsets
//   warp 1     one thread issues 4 k-steps x 2 tcgen05.mma with the weight operand read from TMEM and the
//              activation operand from shared memory (K-major descriptor), then tcgen05.commit -> mma_done[s],
//              which frees the A block, its lo twin and the TMEM weight block
//   warps 2-9  epilogue: tcgen05.ld 32 lanes x 32 columns, store to C or to the split-K scratch
// Measured on [64, 2048] x [2048, 128256] / [2048, 16384] (ring sizes and stages switched off one at a time):
// the depth of the activation / TMEM ring sets the pace (2 blocks 449 / 59 us, 4 blocks 266 / 37 us, 6 blocks -
// all that TMEM holds next to the accumulators - 228 / 34 us), the weight ring needs 4 blocks and gains nothing
// beyond, one converter group is within 5 % of two or three, and with conversion and MMAs switched off entirely
// the loads and barriers alone take 210 / 31 us: the k-block round trip (load, hand-offs through four mbarriers,
// reload), not the arithmetic, bounds the kernel at about 0.5 us per 16 KB of weights per SM.
//
// Every mbarrier wait is bounded: on expiry the thread raises a CTA-wide abort flag, records
// RMLK_ERR_TIMEOUT in the caller's status word, and every role falls through to the common exit where TMEM
// is released.  Every TMA load targets this CTA's own shared memory.
#include <mutex>

#include "matmul_tc_kernel.cuh"

namespace rmlk {
namespace tc {

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    // looked up once per process (function-local static: initialised exactly once, also under concurrent first calls)
    static const EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess)
            return reinterpret_cast<EncodeTiledFn>(p);
        return static_cast<EncodeTiledFn>(nullptr);
    }();
    return fn;
}

static bool make_map_2d(CUtensorMap* map, const void* ptr, uint64_t inner, uint64_t outer, uint32_t box_inner, uint32_t box_outer,
                        CUtensorMapSwizzle swizzle, uint64_t row_pitch = 0) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    const cuuint64_t dims[2] = {inner, outer};
    const cuuint64_t strides[1] = {(row_pitch ? row_pitch : inner) * 4};
    const cuuint32_t box[2] = {box_inner, box_outer};
    const cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT32, 2, const_cast<void*>(ptr), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
              swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <int MT, int SW, int SA, int G, bool PEERS>
static int launch(cudaStream_t st, const CUtensorMap& tmW, const CUtensorMap& tmA, const TcParams& p, dim3 grid) {
    using L = SmemLayout<MT, SW, SA>;
    // The kernel's dynamic shared memory limit is raised once per device; std::call_once makes a thread that arrives
    // during another thread's first call wait for the attribute to be set before it launches.
    static std::once_flag configured[64];
    int dev = 0;
    cudaGetDevice(&dev);
    cudaError_t cfg_err = cudaSuccess;
    if (dev >= 0 && dev < 64)
        std::call_once(configured[dev], [&] {
            cfg_err = cudaFuncSetAttribute(tc_gemm_kernel<MT, SW, SA, G, PEERS>, cudaFuncAttributeMaxDynamicSharedMemorySize, L::TOTAL);
        });
    RMLK_CUDA(cfg_err);
    // launched so that it may be scheduled while the previous kernel of the stream drains (the kernel waits, see
    // dep_wait); with split-K inside a cluster the ksplit CTAs of one tile (grid y) form the cluster
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = dim3(threads_for(G));
    cfg.dynamicSmemBytes = L::TOTAL;
    cfg.stream = st;
    cudaLaunchAttribute at[2];
    unsigned na = 0;
    if (p.cluster_reduce) {
        at[na].id = cudaLaunchAttributeClusterDimension;
        at[na].val.clusterDim.x = 1;
        at[na].val.clusterDim.y = grid.y;
        at[na].val.clusterDim.z = 1;
        na++;
    }
    if (dep_launch_enabled()) {
        at[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        at[na].val.programmaticStreamSerializationAllowed = 1;
        na++;
    }
    cfg.attrs = at;
    cfg.numAttrs = na;
    RMLK_CUDA(cudaLaunchKernelEx(&cfg, tc_gemm_kernel<MT, SW, SA, G, PEERS>, tmW, tmA, p));
    RMLK_CHECK_LAUNCH("tc_gemm_kernel");
    return RMLK_OK;
}

}  // namespace tc

bool tc_enabled() {
    static const bool v = [] {
        const char* e = getenv("RMLK_B200_NO_TC");
        return !(e && e[0] == '1');
    }();
    return v;
}

// Eligibility of the tensor-core path for C[M,N] = A[M,K] x W[K,N].
bool tc_matmul_eligible(int64_t m, int64_t n, int64_t k, const void* a, const void* w, const void* c) {
    return tc_enabled() && m >= 5 && (n % tc::BN == 0) && (k % tc::BK == 0) && k >= tc::BK && aligned_to(a, 16) && aligned_to(w, 16) &&
           aligned_to(c, 16) && n < (1ll << 31) && k < (1ll << 31) && m < (1ll << 31) && ceil_div64(m, 128) <= 65535 &&
           tc::encode_fn() != nullptr;
}

// Largest split-K that is added up inside one thread-block cluster.  Each CTA needs a whole SM (198 KB of
// shared memory), and clusters of 8 such CTAs did not all become resident at once on a B200 (128 CTAs ran as
// two waves, twice the time), while clusters of up to 4 did; wider splits go through the scratch buffer.
// RMLK_B200_TC_CLUSTER_MAX=1..8 overrides the limit; 1 sends every split through the scratch buffer.
static int tc_cluster_max() {
    static const int v = [] {
        const char* e = getenv("RMLK_B200_TC_CLUSTER_MAX");
        const int x = e ? atoi(e) : 4;
        return x < 1 ? 1 : x > 8 ? 8 : x;
    }();
    return v;
}
#define TC_CLUSTER_MAX (tc_cluster_max())

int tc_matmul_plan(int64_t m, int64_t n, int64_t k) {
    const int mt = m <= 64 ? 64 : 128;
    const int64_t tiles = (n / tc::BN) * ceil_div64(m, mt);
    const int64_t k_iters = k / tc::BK;
    int64_t s = sm_count() / tiles;  // fill the GPU with one wave of CTAs, never spill into a second
    const int64_t max_s = k_iters / 8 > 0 ? k_iters / 8 : 1;  // at least 8 k-blocks per split
    if (s > max_s) s = max_s;
    if (s < 1) s = 1;
    // Up to TC_CLUSTER_MAX splits add up on chip (one thread-block cluster per tile); wider ones go through the
    // scratch buffer and a second kernel.  (Snapping a 5- or 6-way split down to a 4-CTA cluster used to win; since
    // the second kernel is scheduled under the tail of the first it no longer does: [64,2048]x[2048,3072] takes
    // 13.4 us as 6 x 24 CTAs + sum against 14.3 us as 24 clusters of 4.)
    // (Capping a wider split at the cluster size for short K was measured and did not pay: [64,2048]x[2048,2048]
    // took 13.9 us as 4-CTA clusters against 11.0 us + a 2-3 us reduction as an 8-way scratch split.)
    return static_cast<int>(s > 32 ? 32 : s);
}

// Scratch for the split-K slabs when the plan splits K more ways than one thread-block cluster adds up.
size_t tc_matmul_workspace_bytes(int64_t m, int64_t n, int64_t k) {
    const int s = tc_matmul_plan(m, n, k);
    return s > TC_CLUSTER_MAX ? static_cast<size_t>(s) * m * n * sizeof(float) : 0;
}

// Launches the tensor-core GEMM.  `ksplit_out` tells the caller how many partial slabs were written to
// `workspace` (1 = the result is already in c).
int tc_matmul(cudaStream_t st, int64_t m, int64_t n, int64_t k, const float* a, const float* w, float* c, void* workspace,
              size_t workspace_bytes, int* status, int* ksplit_out, int flags, int64_t ld, const TcPeers* peers) {
    if (peers && (ld > 0 || peers->n_peer < 0 || peers->n_peer > tc::MAX_PEERS || peers->ldc < n || peers->ldc % 4))
        return fail(RMLK_ERR_INVALID_ARG, "matmul: bad peer destinations");
    const int64_t ldc = peers ? peers->ldc : (ld > 0 ? ld : n);
    const int mt = m <= 64 ? 64 : 128;
    int ksplit = tc_matmul_plan(m, n, k);
    if (ksplit > TC_CLUSTER_MAX && (!workspace || workspace_bytes < static_cast<size_t>(ksplit) * m * n * sizeof(float)))
        ksplit = TC_CLUSTER_MAX;  // no scratch from the caller: one cluster per tile
    const int k_iters = static_cast<int>(k / tc::BK);
    const int per = static_cast<int>(ceil_div64(k_iters, ksplit));
    ksplit = static_cast<int>(ceil_div64(k_iters, per));  // every split gets at least one k-block
    const bool cluster = ksplit > 1 && ksplit <= TC_CLUSTER_MAX;
    CUtensorMap tmW, tmA;
    // ld > 0: w and c are blocks of n columns of matrices whose rows are ld elements apart (no K split in that form)
    if (ld > 0 && ksplit > 1) return fail(RMLK_ERR_INVALID_ARG, "matmul: a column window needs a shape that runs without a K split");
    if (!tc::make_map_2d(&tmW, w, static_cast<uint64_t>(n), static_cast<uint64_t>(k), tc::BN, tc::BK, CU_TENSOR_MAP_SWIZZLE_NONE,
                         ld > 0 ? static_cast<uint64_t>(ld) : 0) ||
        !tc::make_map_2d(&tmA, a, static_cast<uint64_t>(k), static_cast<uint64_t>(m), 32, static_cast<uint32_t>(mt), CU_TENSOR_MAP_SWIZZLE_128B))
        return fail(RMLK_ERR_INTERNAL, "matmul: cuTensorMapEncodeTiled failed");
    tc::TcParams p;
    p.cluster_reduce = cluster ? 1 : 0;
    p.out = (ksplit > 1 && !cluster) ? static_cast<float*>(workspace) : c;
    p.M = m; p.N = n; p.K = k;
    // a split through the scratch leaves dense [ksplit][m][n] slabs; whoever adds them up writes C (and the peers' copies)
    const bool slabs = ksplit > 1 && !cluster;
    p.ldc = slabs ? n : ldc;
    p.n_peer = (peers && !slabs) ? peers->n_peer : 0;
    for (int d = 0; d < p.n_peer; d++) p.peer_out[d] = peers->out[d];
    p.k_iters_per_split = per;
    p.k_iters_total = k_iters;
    p.ksplit = ksplit;
    p.status = status;
    p.w_static = (flags & RMLK_MATMUL_B_STATIC) ? 1 : 0;
    dim3 grid(static_cast<unsigned>(n / tc::BN), static_cast<unsigned>(ksplit), static_cast<unsigned>(ceil_div64(m, mt)));
    *ksplit_out = cluster ? 1 : ksplit;  // slabs left in `workspace` for the caller to add
    if (p.n_peer > 0) {
        if (mt == 64) return tc::launch<64, 4, 6, 2, true>(st, tmW, tmA, p, grid);
        return tc::launch<128, 4, 4, 2, true>(st, tmW, tmA, p, grid);
    }
    // (weight rings of 6 and 8 blocks next to the 6 activation blocks measured 1-3 % slower than 4)
    if (mt == 64) return tc::launch<64, 4, 6, 2, false>(st, tmW, tmA, p, grid);
    return tc::launch<128, 4, 4, 2, false>(st, tmW, tmA, p, grid);
}

}  // namespace rmlk
