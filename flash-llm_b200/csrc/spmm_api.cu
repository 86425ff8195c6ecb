// Host side of libSpMM_API.so: argument checks, launch-plan choice and kernel launches behind the reference's
// SpMM_SplitK_API interface (reference csrc/SpMM_API.cu:22-130), plus the C-linkage aliases.
#include <cuda.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <mutex>
#include <new>

#include "../../include/SpMM_API.cuh"
#include "spmm_kernel_direct_sm100.cuh"
#include "spmm_kernel_sm100.cuh"
#include "tiled_csl_host.h"
#include "tiling.h"

namespace flashllm {

__device__ unsigned int g_status_word = 0;

// Scratch of the allocation-free entry point FlashLLM_SpMM_SplitK_NoAlloc: room for the fp32 partial matrices the
// K split parks between the SpMM kernel and its reduction.  It lives in the library image, so every GPU that loads
// the library carries these 8 MiB until the process exits.  In host code this name is only a handle for
// cudaGetSymbolAddress; the device address obtained from it (once per device) is what the kernels receive.
constexpr size_t kNoAllocScratchBytes = size_t(8) << 20;
static __device__ __align__(256) unsigned char g_noalloc_scratch[kNoAllocScratchBytes];

// Arrival counters of the in-kernel split-K sum: kCounterSets sets of one word per output tile, all zero between
// launches.  Launches of one stream are ordered (the sum of one is over before the next one's B loader is let
// through), so a set is bound to a stream; calls on other streams take other sets, and a call that finds no free
// set, or has more output tiles than a set holds, sums with the second kernel instead.
constexpr int kCounterSets = 32, kCounterTiles = 2048;
static __device__ unsigned int g_tile_counters[kCounterSets * kCounterTiles];

static std::atomic<unsigned long long> g_launches{0};

void count_launch()
{
    g_launches.fetch_add(1, std::memory_order_relaxed);
}

// ---------------------------------------------------------------- per-device state

constexpr int kMaxDevices = 64;

struct DeviceState {
    std::mutex     mutex;
    bool           ready      = false;  // set once every step of the set-up has succeeded; a failed set-up is retried
    int            sm_count   = 0;
    int            smem_optin = 0;
    unsigned int*  status     = nullptr;
    unsigned char* noalloc_scratch = nullptr;  // device address of g_noalloc_scratch on this device
    unsigned int*  tile_counters   = nullptr;  // device address of g_tile_counters on this device
    int            counter_streams = 0;        // streams that own a counter set so far
    cudaStream_t   counter_stream[kCounterSets] = {nullptr};
};

// The counter set of `stream` on this device, or nullptr when all sets are taken by other streams.
static unsigned int* counters_of_stream(DeviceState* st, cudaStream_t stream)
{
    std::lock_guard<std::mutex> lock(st->mutex);
    for (int i = 0; i < st->counter_streams; ++i)
        if (st->counter_stream[i] == stream)
            return st->tile_counters + static_cast<size_t>(i) * kCounterTiles;
    if (st->counter_streams >= kCounterSets)
        return nullptr;
    st->counter_stream[st->counter_streams] = stream;
    return st->tile_counters + static_cast<size_t>(st->counter_streams++) * kCounterTiles;
}

static DeviceState g_devices[kMaxDevices];

using EncodeTiledFn = CUresult (*)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
static EncodeTiledFn  g_encode_tiled = nullptr;
static std::once_flag g_encode_once;

// Register budget of the register-streaming kernel: vectors per lane kept in registers (tiles of up to 768 vectors,
// i.e. 62.5 % sparsity, need no overflow loop), for its two shapes: 8 scatter warps and one CTA per SM; 4 scatter
// warps and two CTAs per SM.
#ifndef FLASHLLM_NARROW_CAP
#define FLASHLLM_NARROW_CAP 14
#endif
#ifndef FLASHLLM_PAIR_CAP
#define FLASHLLM_PAIR_CAP 8
#endif
// ... and of its shape with two warps per tile (4 stages, 8 scatter warps, two CTAs per SM): rows per warp
#ifndef FLASHLLM_DIRECT_BLOCKS
#define FLASHLLM_DIRECT_BLOCKS 2
#endif
constexpr int kDirectBlocks = FLASHLLM_DIRECT_BLOCKS;  // CTAs per SM of the 4-stage shapes
constexpr int kDirectCapWide = 24, kDirectCapNarrow = FLASHLLM_NARROW_CAP, kDirectCapPair = FLASHLLM_PAIR_CAP;

template<typename Kernel>
static cudaError_t raise_smem_limit_of(Kernel kernel, int optin)
{
    cudaFuncAttributes attr{};
    cudaError_t        e = cudaFuncGetAttributes(&attr, kernel);
    if (e != cudaSuccess)
        return e;
    // the opt-in limit covers static and dynamic shared memory together
    return cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                optin - static_cast<int>(attr.sharedSizeBytes));
}

template<int N_TILE>
static cudaError_t raise_smem_limit(int optin)
{
    cudaError_t e = raise_smem_limit_of(spmm_tcgen05_kernel<N_TILE>, optin);
    if (e == cudaSuccess)
        e = raise_smem_limit_of(spmm_tcgen05_direct_kernel<N_TILE, kDirectCapWide, 8, 1>, optin);
    if (e == cudaSuccess)
        e = raise_smem_limit_of(spmm_tcgen05_direct_kernel<N_TILE, kDirectCapNarrow, 4, kDirectBlocks>, optin);
    if (e == cudaSuccess)
        e = raise_smem_limit_of(spmm_tcgen05_direct_kernel<N_TILE, kDirectCapPair, 4, 2, 2>, optin);
    return e;
}

static DeviceState* device_state(cudaError_t* err)
{
    int dev = 0;
    *err    = cudaGetDevice(&dev);
    if (*err != cudaSuccess)
        return nullptr;
    if (dev < 0 || dev >= kMaxDevices) {
        *err = cudaErrorInvalidDevice;
        return nullptr;
    }
    DeviceState* st = &g_devices[dev];
    std::lock_guard<std::mutex> lock(st->mutex);
    if (st->ready) {
        *err = cudaSuccess;
        return st;
    }
    // Nothing here allocates.  A failure (for instance a first call made while a stream is being captured) is
    // returned to this caller only; the next call tries again.
    cudaError_t e = cudaDeviceGetAttribute(&st->sm_count, cudaDevAttrMultiProcessorCount, dev);
    if (e == cudaSuccess)
        e = cudaDeviceGetAttribute(&st->smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    if (e == cudaSuccess)
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st->status), g_status_word);
    if (e == cudaSuccess)
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st->noalloc_scratch), g_noalloc_scratch);
    if (e == cudaSuccess)
        e = cudaGetSymbolAddress(reinterpret_cast<void**>(&st->tile_counters), g_tile_counters);
    // The opt-in limit is a per-device property of each kernel; raise it once instead of on every call
    // (the reference calls cudaFuncSetAttribute per launch, csrc/SpMM_API.cu:36-37).
    if (e == cudaSuccess)
        e = raise_smem_limit<16>(st->smem_optin);
    if (e == cudaSuccess)
        e = raise_smem_limit<32>(st->smem_optin);
    if (e == cudaSuccess)
        e = raise_smem_limit<64>(st->smem_optin);
    if (e == cudaSuccess)
        e = raise_smem_limit<128>(st->smem_optin);
    st->ready = (e == cudaSuccess);
    *err      = e;
    return st->ready ? st : nullptr;
}

int device_status_pointer(unsigned int** status)
{
    cudaError_t  err = cudaSuccess;
    DeviceState* st  = device_state(&err);
    if (!st)
        return static_cast<int>(err);
    *status = st->status;
    return 0;
}

static cudaError_t load_encode_tiled()
{
    std::call_once(g_encode_once, []() {
        void*                           fn = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &qres) == cudaSuccess
            && qres == cudaDriverEntryPointSuccess)
            g_encode_tiled = reinterpret_cast<EncodeTiledFn>(fn);
    });
    return g_encode_tiled ? cudaSuccess : cudaErrorNotSupported;
}

// ---------------------------------------------------------------- launch plan

struct PlanOverride {
    int v[kPlanFieldCount] = {0};
};
static PlanOverride g_override;
static std::mutex   g_override_mutex;
static std::atomic<int> g_launch_overlap{0};


constexpr int kDefaultPath = kPathDirect;

static int n_tile_for(int N)
{
    return N <= 16 ? 16 : (N <= 32 ? 32 : (N <= 64 ? 64 : 128));
}

static int plan_smem_bytes(const SpmmPlan& pl)
{
    const int bars = 8 * (2 * pl.ring_slots + 2 * pl.a_stages + 2 * pl.b_stages + 1) + 16 + 4 * pl.offsets_staged;
    return pl.a_stages * kDenseTileBytes + pl.b_stages * pl.b_batch * pl.n_tile * kTileK * 2
           + pl.ring_slots * pl.chunk_vectors * 16 + bars;
}

static bool is_pow2(int v)
{
    return v > 0 && (v & (v - 1)) == 0;
}

// Chooses how to cut K and how deep to pipeline.  Takes the place of the reference's per-N switch over
// TilingConfig instances (csrc/SpMM_API.cu:79-118) and of its hand-tuned Split_K tables
// (kernel_benchmark/benchmark.sh:13-15).
// `max_parts`: workspace parts the caller has room for (Split_K / 2 for a caller's Reduction_Workspace, whose Split_K
// fp16 matrices hold half as many fp32 ones).
// `sends`: the call is the sending half of a fused all-reduce, where workspace parts are always summed by the last
// CTA of a tile, which then also stores the sum to every GPU.
static cudaError_t make_plan(const DeviceState* st, int M, int N, int K, int max_parts, SpmmPlan* out, bool sends = false)
{
    PlanOverride ov;
    {
        std::lock_guard<std::mutex> lock(g_override_mutex);
        ov = g_override;
    }
    SpmmPlan pl{};
    pl.n_tile           = n_tile_for(N);
    const int tile_rows = M / kTileM;
    const int k_tiles   = K / kTileK;
    const int n_tiles   = (N + pl.n_tile - 1) / pl.n_tile;
    const int ctas_flat = tile_rows * n_tiles;
    const int slab      = pl.n_tile * kTileK * 2;

    // Two pipelines per SM (4 scatter warps, 4 stages each) where they fit; wide-N tiles need the shared memory for
    // their B batches, so they run one deeper pipeline per SM instead.
    pl.path               = ov.v[kPlanPath] ? ov.v[kPlanPath] : kDefaultPath;
    const bool direct     = pl.path == kPathDirect;
    pl.scatter_warps      = ov.v[kPlanScatterWarps] ? ov.v[kPlanScatterWarps]
                                                    : (direct ? (pl.n_tile <= 64 ? 4 : 8) : (pl.n_tile <= 32 ? 4 : 8));
    const bool two_per_sm = direct ? pl.scatter_warps < 8 : pl.n_tile <= 32;
    pl.producers       = ov.v[kPlanProducers] ? ov.v[kPlanProducers] : 1;
    pl.chunk_vectors   = ov.v[kPlanChunkVectors] ? ov.v[kPlanChunkVectors] : 512;
    pl.ring_slots      = ov.v[kPlanRingSlots] ? ov.v[kPlanRingSlots]
                                              : (two_per_sm ? kMaxTileVectors / pl.chunk_vectors + 1 : 8);
    if (!ov.v[kPlanRingSlots])
        pl.ring_slots = (pl.ring_slots + pl.producers - 1) / pl.producers * pl.producers;
    pl.a_stages        = ov.v[kPlanAStages] ? ov.v[kPlanAStages] : pl.scatter_warps;
    pl.b_batch         = ov.v[kPlanBBatch] ? ov.v[kPlanBBatch] : (4096 / slab > 0 ? 4096 / slab : 1);
    pl.b_stages        = ov.v[kPlanBStages] ? ov.v[kPlanBStages] : 2;
    if (direct) {  // one stage per scatter warp, no copy ring; B batches split evenly between the MMA issuers
        if (!ov.v[kPlanBBatch])
            pl.b_batch = (pl.b_batch + kDirectIssuers - 1) / kDirectIssuers * kDirectIssuers;
        pl.a_stages      = pl.scatter_warps;
        // `producers` of the register-streaming form = warps that share one tile (1, or 2 with four stages)
        pl.producers     = (ov.v[kPlanProducers] == 2 && pl.scatter_warps == 4) ? 2 : 1;
        pl.ring_slots    = 0;
        pl.chunk_vectors = 0;
    }
    // How to cut K.  A CTA that owns a whole tile row needs no reduction and pays its set-up and pipeline fill once,
    // so K is cut only to fill the GPU.  S parts are summed inside a thread-block cluster (distributed shared memory),
    // G parts through fp32 partial tiles in the workspace (summed by the last CTA of a tile to finish, or by a second
    // kernel).  A launch of rows*G clusters of S CTAs runs in ceil(rows*G / capacity(S)) waves, where capacity(S) is
    // the number of clusters of S CTAs the GPU holds at a time -- measured, and well below slots/S for S >= 3 (71
    // clusters of 4, 33 of 8 on 296 slots): one cluster more than that and the launch takes twice as long.  Every
    // CTA processes k_tiles/(S*G) tiles after a fixed cost worth about 16 tiles; a cluster sum costs about 3 more,
    // the sum by the last CTA 2 + 0.1 per part (8 + 0.1 per part in a fused all-reduce, where the peers wait for that
    // CTA: measured on 2 GPUs, 9216x1152 ... 9216x18432), a second kernel half a tile per part.  The cheapest (S, G) wins,
    // fewer parts on a tie.  Replaces the reference's hand-tuned Split_K tables (kernel_benchmark/benchmark.sh:13-15).
    static const int kClustersResident2[kMaxClusterK + 1] = {0, 296, 148, 92, 71, 56, 45, 37, 33};  // two CTAs per SM
    static const int kClustersResident1[kMaxClusterK + 1] = {0, 148, 74, 45, 33, 26, 22, 15, 15};   // one CTA per SM
    const bool two_resident = two_per_sm && ((direct && pl.producers == 1) ? kDirectBlocks : 2) == 2;
    const int* resident     = two_resident ? kClustersResident2 : kClustersResident1;
    auto capacity = [&](int S_) {  // the table is for 148 SMs
        const long long c = static_cast<long long>(resident[S_]) * st->sm_count / 148;
        return c < 1 ? 1ll : c;
    };
    const int max_extra = max_parts > 1 ? max_parts : 1;
    // (measured on eleven shapes from 9216x1152 to 9216x36864: with launch overlap the second kernel hides behind its
    // neighbours and beats the sum by the last CTA, which sits on every tile's critical path, by ~2 us per call;
    // without overlap the two are level.  The fused all-reduce always sums by the last CTA: that CTA also sends.)
    pl.reduce           = sends ? kReduceLastCta : (ov.v[kPlanReduce] ? ov.v[kPlanReduce] : kReduceSecondKernel);
    if (ctas_flat > kCounterTiles)
        pl.reduce = kReduceSecondKernel;
    // (without launch overlap a second kernel costs a whole launch: small problems then do better with clusters alone)
    const bool no_second = pl.reduce == kReduceSecondKernel && static_cast<long long>(tile_rows) * k_tiles <= 4096
                           && g_launch_overlap.load(std::memory_order_relaxed) == 0;
    int    best_s = 1, best_g = 1;
    double best_cost = 0.0;
    for (int s_ = 1; s_ <= kMaxClusterK && s_ <= k_tiles; ++s_) {
        for (int g = 1; g <= max_extra && g <= 32 && s_ * g <= k_tiles; ++g) {
            if (g > 1 && no_second)
                break;
            const long long clusters = static_cast<long long>(ctas_flat) * g;
            const double    waves    = static_cast<double>((clusters + capacity(s_) - 1) / capacity(s_));
            const double    per_cta  = static_cast<double>((k_tiles + s_ * g - 1) / (s_ * g)) + 16.0 + (s_ > 1 ? 3.0 : 0.0)
                                    + (g > 1 && pl.reduce == kReduceLastCta ? (sends ? 8.0 : 2.0) + 0.1 * g : 0.0);
            const double cost = waves * per_cta + (g > 1 && pl.reduce == kReduceSecondKernel ? 0.5 * g : 0.0);
            if ((s_ == 1 && g == 1) || cost < best_cost - 1e-9
                || (cost < best_cost + 1e-9 && s_ * g < best_s * best_g)) {
                best_cost = cost;
                best_s    = s_;
                best_g    = g;
            }
        }
    }
    pl.cluster_k = ov.v[kPlanClusterK] ? ov.v[kPlanClusterK] : best_s;
    if (pl.cluster_k > k_tiles)
        pl.cluster_k = k_tiles;
    int extra = ov.v[kPlanWorkspaceK] ? ov.v[kPlanWorkspaceK] : best_g;
    if (extra > max_extra)
        extra = max_extra;  // the workspace is promised to hold Split_K fp16 matrices = Split_K/2 fp32 partials
    if (extra * pl.cluster_k > k_tiles)
        extra = k_tiles / pl.cluster_k;
    if (extra < 1)
        extra = 1;
    pl.workspace_k = extra;
    // room for this CTA's slice of TileOffsets (K tiles of the longest part, plus one), up to 8 KB
    const int longest = (k_tiles + pl.cluster_k * pl.workspace_k - 1) / (pl.cluster_k * pl.workspace_k) + 1;
    pl.offsets_staged = longest + 1 <= 2048 ? ((longest + 1 + 3) / 4) * 4 : 0;
    pl.smem_bytes     = plan_smem_bytes(pl);

    const bool ring_ok = pl.scatter_warps >= 4 && pl.scatter_warps <= kMaxScatterWarps
                         && pl.producers >= 1 && pl.producers <= kMaxProducers && is_pow2(pl.chunk_vectors)
                         && pl.chunk_vectors >= 64 && pl.ring_slots <= kMaxRingSlots
                         // a slot is always refilled by the same producer warp, and a stage's successive tiles are
                         // taken by groups that cannot be two uses ahead: both keep every mbarrier parity wait within
                         // one phase
                         && pl.ring_slots % pl.producers == 0 && pl.a_stages >= pl.scatter_warps
                         && pl.ring_slots * pl.chunk_vectors >= kMaxTileVectors + pl.chunk_vectors;
    const bool direct_ok = (pl.scatter_warps == 4 || pl.scatter_warps == 8)
                           && pl.a_stages == pl.scatter_warps && pl.b_batch % kDirectIssuers == 0;
    const bool ok = (pl.path == kPathRing || pl.path == kPathDirect) && (direct ? direct_ok : ring_ok)
                    && pl.a_stages >= 1 && pl.a_stages <= kMaxAStages && pl.b_stages >= 1 && pl.b_stages <= kMaxBStages
                    && pl.b_batch >= 1 && pl.b_batch <= 256 && pl.cluster_k >= 1 && pl.cluster_k <= kMaxClusterK
                    && pl.workspace_k >= 1 && (pl.reduce == kReduceSecondKernel || pl.reduce == kReduceLastCta)
                    && pl.smem_bytes <= st->smem_optin
                    // the fp32 partial tile of the cluster reduction is parked over the pipeline buffers
                    && pl.smem_bytes - 1024 - 4 * pl.offsets_staged >= pl.n_tile * kTileM * 4;
    if (!ok)
        return cudaErrorInvalidConfiguration;
    *out = pl;
    return cudaSuccess;
}

template<int N_TILE>
static cudaError_t launch_spmm(cudaStream_t stream, const CUtensorMap& tmap, const SpmmParams& params, int tile_rows,
                               int n_tiles)
{
    const SpmmPlan&     pl = params.plan;
    cudaLaunchConfig_t  cfg{};
    cudaLaunchAttribute attr[2];
    cfg.gridDim          = dim3(pl.cluster_k, tile_rows, n_tiles * pl.workspace_k);
    cfg.blockDim         = dim3((pl.path == kPathDirect ? 1 + kDirectIssuers + pl.scatter_warps * pl.producers
                                                        : pl.producers + 2 + pl.scatter_warps) * 32, 1, 1);
    cfg.dynamicSmemBytes = pl.smem_bytes;
    cfg.stream           = stream;
    attr[0].id               = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = pl.cluster_k;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs                = attr;
    cfg.numAttrs             = 1;
    if (g_launch_overlap.load(std::memory_order_relaxed)) {
        attr[1].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.numAttrs                                       = 2;
    }
    count_launch();
    if (pl.path == kPathDirect) {
        if (pl.scatter_warps == 8)
            return cudaLaunchKernelEx(&cfg, spmm_tcgen05_direct_kernel<N_TILE, kDirectCapWide, 8, 1>, tmap, params);
        if (pl.producers == 2)
            return cudaLaunchKernelEx(&cfg, spmm_tcgen05_direct_kernel<N_TILE, kDirectCapPair, 4, 2, 2>, tmap, params);
        return cudaLaunchKernelEx(&cfg, spmm_tcgen05_direct_kernel<N_TILE, kDirectCapNarrow, 4, kDirectBlocks>, tmap, params);
    }
    return cudaLaunchKernelEx(&cfg, spmm_tcgen05_kernel<N_TILE>, tmap, params);
}

static cudaError_t reduce_partials(cudaStream_t stream, half* C, const float* ws, long long count, int parts,
                                   const half* bias, int M, int activation, const half* residual)
{
    const int       threads = 256;
    const long long groups  = (count + 3) / 4;
    const unsigned  blocks  = static_cast<unsigned>((groups + threads - 1) / threads);
    count_launch();
    cudaLaunchConfig_t  cfg{};
    cudaLaunchAttribute attr[1];
    cfg.gridDim  = dim3(blocks, 1, 1);
    cfg.blockDim = dim3(threads, 1, 1);
    cfg.stream   = stream;
    if (g_launch_overlap.load(std::memory_order_relaxed)) {
        attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[0].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs                                          = attr;
        cfg.numAttrs                                       = 1;
    }
    return cudaLaunchKernelEx(&cfg, splitk_reduce_f32_kernel, C, ws, count, parts, bias, M, activation, residual);
}

static cudaError_t reduce_workspace(cudaStream_t stream, half* C, const half* ws, long long count, int parts)
{
    const int       threads = 256;
    const long long groups  = (count + 7) / 8;
    const unsigned  blocks  = static_cast<unsigned>((groups + threads - 1) / threads);
    count_launch();
    splitk_reduce_kernel<<<blocks, threads, 0, stream>>>(C, ws, count, parts);
    return cudaGetLastError();
}

static bool n_supported(int N)
{
    // the reference's dispatch list (csrc/SpMM_API.cu:79-118)
    return N == 8 || N == 16 || N == 32 || N == 64 || (N > 0 && N % 128 == 0);
}

}  // namespace flashllm

using namespace flashllm;

// Receive buffers of a GPU group for the fused row-parallel SpMM + all-reduce.  Every GPU owns one buffer with two
// sets (used by alternate calls) of `world` fp32 slots [max_elems] and `world` x kCommFlagsPerRank flag words:
//   [set 0 slots][set 1 slots][set 0 flags][set 1 flags][own partial matrices][own arrival counters]
// Slot w / flag row w of a GPU's buffer is written only by GPU w.  While one call's sums are still being read on a
// slow GPU, a fast GPU's next call writes the other set; it cannot start the call after that before the slow GPU has
// taken part in the next one, so two sets are enough.
constexpr int kCommFlagsPerRank = 8192;

struct FlashLLMComm {
    int            rank = 0, world = 0;
    long long      max_elems = 0;
    unsigned char* buffer[kMaxPushWorld] = {nullptr};  // buffer[w]: GPU w's receive buffer as mapped in this process
    unsigned int   epoch = 0;                          // calls made so far; every GPU of the group makes the same calls
    // How long the summing kernel waits for the slowest GPU of the group before it gives up (status bit 32).  The
    // GPUs of a group enter a layer at slightly different times; the limit only has to end a wait for a partner that
    // never comes.
    unsigned long long wait_limit_ns = 2000ull * 1000ull * 1000ull;
};

static size_t comm_slot_bytes(int world, long long max_elems)
{
    return static_cast<size_t>(world) * static_cast<size_t>(max_elems) * sizeof(float);
}

static size_t comm_flag_bytes(int world)
{
    return static_cast<size_t>(world) * kCommFlagsPerRank * sizeof(unsigned int);
}

// ... followed by what only the owning GPU touches: room for kCommLocalParts fp32 partial matrices of its own K
// split, and the arrival counters of that split's in-kernel sum (zero between calls).
constexpr int kCommLocalParts = 8, kCommCounterTiles = 4096;

static size_t comm_buffer_bytes(int world, long long max_elems)
{
    return 2 * comm_slot_bytes(world, max_elems) + 2 * comm_flag_bytes(world)
           + kCommLocalParts * static_cast<size_t>(max_elems) * sizeof(float) + kCommCounterTiles * sizeof(unsigned int);
}

// SpMM_SplitK_API plus the output epilogue (bias of output feature m, activation) the public entry points select.
static cudaError_t spmm_launch_all(cudaStream_t stream,
                                   const uint4* Compressed_A,
                                   const int*   TileOffsets,
                                   const half*  B,
                                   half*        C,
                                   const int    M_Global,
                                   const int    N_Global,
                                   const int    K_Global,
                                   half*        Reduction_Workspace,
                                   int          Split_K,
                                   const half*  bias,
                                   int          activation,
                                   const half*  residual = nullptr,
                                   FlashLLMComm* comm = nullptr,
                                   int           phases = 3)
{
    if (!n_supported(N_Global)) {
        printf("MM_Sparse_API Error: Unsupported N dimension %d!\n", N_Global);
        return cudaErrorUnknown;
    }
    if (M_Global <= 0 || K_Global <= 0 || M_Global % kTileM != 0 || K_Global % kTileK != 0 || Split_K < 1
        || Compressed_A == nullptr || TileOffsets == nullptr || B == nullptr || C == nullptr
        || (reinterpret_cast<uintptr_t>(Compressed_A) & 15u) != 0 || (reinterpret_cast<uintptr_t>(B) & 15u) != 0
        || (reinterpret_cast<uintptr_t>(C) & 1u) != 0 || (Split_K > 1 && Reduction_Workspace == nullptr))
        return cudaErrorInvalidValue;

    cudaError_t  err = cudaSuccess;
    DeviceState* st  = device_state(&err);
    if (!st)
        return err;
    if ((err = load_encode_tiled()) != cudaSuccess)
        return err;

    SpmmParams params{};
    if ((err = make_plan(st, M_Global, N_Global, K_Global, comm ? kCommLocalParts : Split_K / 2, &params.plan,
                         comm != nullptr))
        != cudaSuccess)
        return err;
    SpmmPlan& pl = params.plan;
    // The sum over workspace parts reads 16-byte groups of the workspace and writes 8-byte groups of C.
    if (!comm && pl.workspace_k > 1
        && ((reinterpret_cast<uintptr_t>(Reduction_Workspace) & 15u) != 0 || (reinterpret_cast<uintptr_t>(C) & 7u) != 0))
        pl.workspace_k = 1;

    params.compressed   = Compressed_A;
    params.tile_offsets = TileOffsets;
    params.out          = C;
    params.partial      = pl.workspace_k > 1 ? reinterpret_cast<float*>(Reduction_Workspace) : nullptr;
    if (!comm && pl.workspace_k > 1 && pl.reduce == kReduceLastCta) {
        params.tile_counters = counters_of_stream(st, stream);
        if (params.tile_counters == nullptr)
            pl.reduce = kReduceSecondKernel;  // every counter set belongs to another stream
    }
    params.status       = st->status;
    params.bias         = bias;
    params.activation   = activation;
    params.residual     = residual;
    params.M            = M_Global;
    params.N            = N_Global;
    params.K            = K_Global;
    params.k_tiles      = K_Global / kTileK;

    // B as a 3-D tensor {64 K-elements (inner), N, K/64}: one box = b_batch K tiles of [n_tile x 64], each stored as
    // a 128-byte-swizzled slab; rows past N and K tiles past K/64 read as 0.
    CUtensorMap      tmap;
    const cuuint64_t dims[3]    = {static_cast<cuuint64_t>(kTileK), static_cast<cuuint64_t>(N_Global),
                                   static_cast<cuuint64_t>(K_Global / kTileK)};
    const cuuint64_t strides[2] = {static_cast<cuuint64_t>(K_Global) * 2, static_cast<cuuint64_t>(kTileK) * 2};
    const cuuint32_t box[3]     = {static_cast<cuuint32_t>(kTileK), static_cast<cuuint32_t>(pl.n_tile),
                                   static_cast<cuuint32_t>(pl.b_batch)};
    const cuuint32_t estr[3]    = {1, 1, 1};
    const CUresult   cres       = g_encode_tiled(&tmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<half*>(B), dims,
                                       strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cres != CUDA_SUCCESS)
        return cudaErrorInvalidValue;

    const int tile_rows = M_Global / kTileM;
    const int n_tiles   = (N_Global + pl.n_tile - 1) / pl.n_tile;
    const int grid_ctas = pl.cluster_k * tile_rows * n_tiles * pl.workspace_k;
    // flags a sender raises per call: one per CTA, or one per output tile when the last CTA of a tile sends its sum
    const int comm_flags = pl.workspace_k > 1 ? tile_rows * n_tiles : grid_ctas;
    size_t    set_slots = 0, set_flags = 0;
    if (comm) {
        const long long elems = static_cast<long long>(M_Global) * N_Global;
        if (elems > comm->max_elems || elems % 4 != 0 || comm_flags > kCommFlagsPerRank
            || (pl.workspace_k > 1 && tile_rows * n_tiles > kCommCounterTiles) || (reinterpret_cast<uintptr_t>(C) & 7u) != 0)
            return cudaErrorInvalidValue;
        if (pl.workspace_k > 1) {  // own K split: parts parked in the own buffer, summed and sent by the last CTA
            unsigned char* own   = comm->buffer[comm->rank] + 2 * comm_slot_bytes(comm->world, comm->max_elems)
                                 + 2 * comm_flag_bytes(comm->world);
            pl.reduce            = kReduceLastCta;
            params.partial       = reinterpret_cast<float*>(own);
            params.tile_counters = reinterpret_cast<unsigned int*>(own + kCommLocalParts * static_cast<size_t>(comm->max_elems)
                                                                                 * sizeof(float));
        }
        if (phases & 1)
            comm->epoch += 1;  // a new call; a sum-only call belongs to the call whose stores went out last
        const int set       = static_cast<int>(comm->epoch & 1u);
        set_slots           = static_cast<size_t>(set) * comm_slot_bytes(comm->world, comm->max_elems);
        set_flags           = 2 * comm_slot_bytes(comm->world, comm->max_elems)
                    + static_cast<size_t>(set) * comm_flag_bytes(comm->world);
        params.push_world   = comm->world;
        params.push_epoch   = comm->epoch;
        for (int w = 0; w < comm->world; ++w) {
            params.push_slot[w] = reinterpret_cast<float*>(comm->buffer[w] + set_slots) + comm->rank * comm->max_elems;
            params.push_flag[w] = reinterpret_cast<unsigned int*>(comm->buffer[w] + set_flags) + comm->rank * kCommFlagsPerRank;
        }
    }
    if (!comm || (phases & 1)) {
        switch (pl.n_tile) {
            case 16: err = launch_spmm<16>(stream, tmap, params, tile_rows, n_tiles); break;
            case 32: err = launch_spmm<32>(stream, tmap, params, tile_rows, n_tiles); break;
            case 64: err = launch_spmm<64>(stream, tmap, params, tile_rows, n_tiles); break;
            default: err = launch_spmm<128>(stream, tmap, params, tile_rows, n_tiles); break;
        }
        if (err != cudaSuccess)
            return err;
    }
    if (comm && !(phases & 2))
        return cudaSuccess;
    if (comm) {
        // second kernel: waits (bounded) for every GPU's flags of this call, then adds the slots up in rank order
        const long long     count   = static_cast<long long>(M_Global) * N_Global;
        const int           threads = 256;
        const unsigned      blocks  = static_cast<unsigned>((count / 4 + threads - 1) / threads);
        cudaLaunchConfig_t  cfg{};
        cudaLaunchAttribute attr[1];
        cfg.gridDim  = dim3(blocks, 1, 1);
        cfg.blockDim = dim3(threads, 1, 1);
        cfg.stream   = stream;
        if (g_launch_overlap.load(std::memory_order_relaxed)) {
            attr[0].id                                         = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.attrs                                          = attr;
            cfg.numAttrs                                       = 1;
        }
        unsigned char* mine = comm->buffer[comm->rank];
        count_launch();
        return cudaLaunchKernelEx(&cfg, allreduce_sum_kernel, C, reinterpret_cast<const float*>(mine + set_slots),
                                  comm->max_elems, reinterpret_cast<const unsigned int*>(mine + set_flags), kCommFlagsPerRank,
                                  comm->epoch, comm->world, pl.workspace_k > 1 ? 1 : pl.cluster_k, tile_rows, pl.n_tile, count, bias,
                                  M_Global, activation, residual, st->status, comm->wait_limit_ns, phases == 3 ? 0 : 1);
    }
    if (pl.workspace_k > 1 && pl.reduce == kReduceSecondKernel)
        return reduce_partials(stream, C, params.partial, static_cast<long long>(M_Global) * N_Global, pl.workspace_k,
                               bias, M_Global, activation, residual);
    return cudaSuccess;
}

cudaError_t SpMM_SplitK_API(cudaStream_t stream,
                            const half*  A,
                            const uint4* Compressed_A,
                            const int*   TileOffsets,
                            const half*  B,
                            half*        C,
                            const int    M_Global,
                            const int    N_Global,
                            const int    K_Global,
                            half*        Reduction_Workspace,
                            int          Split_K)
{
    (void)A;  // kept for signature compatibility; callers pass nullptr
    return spmm_launch_all(stream, Compressed_A, TileOffsets, B, C, M_Global, N_Global, K_Global, Reduction_Workspace,
                           Split_K, nullptr, kActNone);
}

extern "C" {

int FlashLLM_SpMM_SplitK_BiasAct(void*       stream,
                                 const void* Compressed_A,
                                 const int*  TileOffsets,
                                 const void* B,
                                 void*       C,
                                 int         M,
                                 int         N,
                                 int         K,
                                 void*       Reduction_Workspace,
                                 int         Split_K,
                                 const void* bias,
                                 int         activation)
{
    if (activation != kActNone && activation != kActRelu)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(spmm_launch_all(static_cast<cudaStream_t>(stream), static_cast<const uint4*>(Compressed_A),
                                            TileOffsets, static_cast<const half*>(B), static_cast<half*>(C), M, N, K,
                                            static_cast<half*>(Reduction_Workspace), Split_K,
                                            static_cast<const half*>(bias), activation));
}

int FlashLLM_SpMM_SplitK_Epilogue(void*       stream,
                                  const void* Compressed_A,
                                  const int*  TileOffsets,
                                  const void* B,
                                  void*       C,
                                  int         M,
                                  int         N,
                                  int         K,
                                  void*       Reduction_Workspace,
                                  int         Split_K,
                                  const void* bias,
                                  int         activation,
                                  const void* residual)
{
    if ((activation != kActNone && activation != kActRelu) || (residual != nullptr && residual == C))
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(spmm_launch_all(static_cast<cudaStream_t>(stream), static_cast<const uint4*>(Compressed_A),
                                            TileOffsets, static_cast<const half*>(B), static_cast<half*>(C), M, N, K,
                                            static_cast<half*>(Reduction_Workspace), Split_K,
                                            static_cast<const half*>(bias), activation,
                                            static_cast<const half*>(residual)));
}

int FlashLLM_SpMM_SplitK(void*       stream,
                         const void* A,
                         const void* Compressed_A,
                         const int*  TileOffsets,
                         const void* B,
                         void*       C,
                         int         M,
                         int         N,
                         int         K,
                         void*       Reduction_Workspace,
                         int         Split_K)
{
    return static_cast<int>(SpMM_SplitK_API(static_cast<cudaStream_t>(stream),
                                            static_cast<const half*>(A),
                                            static_cast<const uint4*>(Compressed_A),
                                            TileOffsets,
                                            static_cast<const half*>(B),
                                            static_cast<half*>(C),
                                            M,
                                            N,
                                            K,
                                            static_cast<half*>(Reduction_Workspace),
                                            Split_K));
}

int FlashLLM_SpMM_SplitK_NoAlloc(void*       stream,
                                 const void* Compressed_A,
                                 const int*  TileOffsets,
                                 const void* B,
                                 void*       C,
                                 int         M,
                                 int         N,
                                 int         K,
                                 int         Split_K)
{
    if (M <= 0 || N <= 0 || K <= 0 || Split_K < 1)
        return static_cast<int>(cudaErrorInvalidValue);
    // Split_K fp16 matrices, the room a caller-owned workspace would have; Split_K = 1 never touches the scratch
    const unsigned long long need = Split_K > 1 ? 2ull * static_cast<unsigned long long>(Split_K) * M * N : 0ull;
    if (need > kNoAllocScratchBytes) {
        fprintf(stderr,
                "FlashLLM_SpMM_SplitK_NoAlloc: Split_K*M*N*2 = %llu bytes exceeds the built-in %zu-byte scratch; lower "
                "Split_K (Split_K = 1 needs no scratch and is accepted at any size) or use FlashLLM_SpMM_SplitK with a "
                "workspace of your own.\n",
                need, kNoAllocScratchBytes);
        return static_cast<int>(cudaErrorInvalidValue);
    }
    cudaError_t  err = cudaSuccess;
    DeviceState* st  = device_state(&err);  // first call on a device: looks the scratch address up, allocates nothing
    if (!st)
        return static_cast<int>(err);
    return static_cast<int>(SpMM_SplitK_API(static_cast<cudaStream_t>(stream), nullptr,
                                            static_cast<const uint4*>(Compressed_A), TileOffsets,
                                            static_cast<const half*>(B), static_cast<half*>(C), M, N, K,
                                            reinterpret_cast<half*>(st->noalloc_scratch), Split_K));
}

unsigned long long FlashLLM_Comm_BufferBytes(int world, long long max_elems)
{
    if (world < 1 || world > kMaxPushWorld || max_elems < 4)
        return 0;
    return comm_buffer_bytes(world, max_elems);
}

int FlashLLM_Comm_AllocBuffer(int world, long long max_elems, void** buffer, void* ipc_handle)
{
    if (buffer == nullptr || world < 1 || world > kMaxPushWorld || max_elems < 4 || max_elems % 4 != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    const size_t bytes = comm_buffer_bytes(world, max_elems);
    cudaError_t  e     = cudaMalloc(buffer, bytes);
    if (e == cudaSuccess)
        e = cudaMemset(*buffer, 0, bytes);  // flags start below every epoch
    if (e == cudaSuccess && ipc_handle != nullptr)
        e = cudaIpcGetMemHandle(static_cast<cudaIpcMemHandle_t*>(ipc_handle), *buffer);
    if (e == cudaSuccess)
        e = cudaDeviceSynchronize();
    return static_cast<int>(e);
}

int FlashLLM_Comm_OpenPeerBuffer(const void* ipc_handle, void** buffer)
{
    if (ipc_handle == nullptr || buffer == nullptr)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(cudaIpcOpenMemHandle(buffer, *static_cast<const cudaIpcMemHandle_t*>(ipc_handle),
                                                 cudaIpcMemLazyEnablePeerAccess));
}

int FlashLLM_Comm_ClosePeerBuffer(void* buffer)
{
    return static_cast<int>(cudaIpcCloseMemHandle(buffer));
}

int FlashLLM_Comm_FreeBuffer(void* buffer)
{
    return static_cast<int>(cudaFree(buffer));
}

int FlashLLM_Comm_Create(void** comm, int rank, int world, long long max_elems, void* const* buffers)
{
    if (comm == nullptr || buffers == nullptr || world < 1 || world > kMaxPushWorld || rank < 0 || rank >= world
        || max_elems < 4 || max_elems % 4 != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    for (int w = 0; w < world; ++w)
        if (buffers[w] == nullptr || (reinterpret_cast<uintptr_t>(buffers[w]) & 15u) != 0)
            return static_cast<int>(cudaErrorInvalidValue);
    FlashLLMComm* c = new (std::nothrow) FlashLLMComm();
    if (c == nullptr)
        return static_cast<int>(cudaErrorMemoryAllocation);
    c->rank      = rank;
    c->world     = world;
    c->max_elems = max_elems;
    for (int w = 0; w < world; ++w)
        c->buffer[w] = static_cast<unsigned char*>(buffers[w]);
    *comm = c;
    return 0;
}

int FlashLLM_Comm_SetWaitLimit(void* comm, int milliseconds)
{
    if (comm == nullptr || milliseconds < 1 || milliseconds > 60000)
        return static_cast<int>(cudaErrorInvalidValue);
    static_cast<FlashLLMComm*>(comm)->wait_limit_ns = static_cast<unsigned long long>(milliseconds) * 1000000ull;
    return 0;
}

int FlashLLM_Comm_Destroy(void* comm)
{
    delete static_cast<FlashLLMComm*>(comm);
    return 0;
}

int FlashLLM_SpMM_SplitK_AllReduce(void*       comm,
                                   void*       stream,
                                   const void* Compressed_A,
                                   const int*  TileOffsets,
                                   const void* B,
                                   void*       C,
                                   int         M,
                                   int         N,
                                   int         K,
                                   const void* bias,
                                   int         activation,
                                   const void* residual,
                                   int         phases)
{
    if (comm == nullptr || (activation != kActNone && activation != kActRelu) || phases < 1 || phases > 3
        || (residual != nullptr && residual == C))
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(spmm_launch_all(static_cast<cudaStream_t>(stream), static_cast<const uint4*>(Compressed_A),
                                            TileOffsets, static_cast<const half*>(B), static_cast<half*>(C), M, N, K,
                                            nullptr, 1, static_cast<const half*>(bias), activation,
                                            static_cast<const half*>(residual), static_cast<FlashLLMComm*>(comm), phases));
}

int FlashLLM_SplitK_Reduction(void* stream, void* C, const void* Reduction_Workspace, int M, int N, int Split_K)
{
    const long long count = static_cast<long long>(M) * N;
    if (C == nullptr || Reduction_Workspace == nullptr || M <= 0 || N <= 0 || Split_K < 1 || count % 8 != 0
        || (reinterpret_cast<uintptr_t>(C) & 15u) != 0 || (reinterpret_cast<uintptr_t>(Reduction_Workspace) & 15u) != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    return static_cast<int>(reduce_workspace(static_cast<cudaStream_t>(stream), static_cast<half*>(C),
                                             static_cast<const half*>(Reduction_Workspace), count, Split_K));
}

void FlashLLM_SetLaunchOverlap(int enable)
{
    g_launch_overlap.store(enable ? 1 : 0, std::memory_order_relaxed);
}

void FlashLLM_SetPlan(const int* fields, int count)
{
    std::lock_guard<std::mutex> lock(g_override_mutex);
    for (int i = 0; i < kPlanFieldCount; ++i)
        g_override.v[i] = (fields != nullptr && i < count) ? fields[i] : 0;
}

int FlashLLM_GetPlan(int M, int N, int K, int Split_K, int* out, int count)
{
    if (out == nullptr || !n_supported(N) || M <= 0 || K <= 0 || M % kTileM != 0 || K % kTileK != 0 || Split_K < 1)
        return static_cast<int>(cudaErrorInvalidValue);
    cudaError_t  err = cudaSuccess;
    DeviceState* st  = device_state(&err);
    if (!st)
        return static_cast<int>(err);
    SpmmPlan pl{};
    if ((err = make_plan(st, M, N, K, Split_K / 2, &pl)) != cudaSuccess)
        return static_cast<int>(err);
    const int values[kPlanFieldCount + 1] = {pl.cluster_k,  pl.workspace_k,   pl.a_stages,      pl.b_stages,  pl.b_batch,
                                             pl.ring_slots, pl.chunk_vectors, pl.scatter_warps, pl.producers, pl.path,
                                             pl.reduce,     pl.smem_bytes};
    for (int i = 0; i < count && i <= kPlanFieldCount; ++i)
        out[i] = values[i];
    return 0;
}

unsigned int FlashLLM_ConsumeStatus(void)
{
    cudaError_t  err = cudaSuccess;
    DeviceState* st  = device_state(&err);
    if (!st)
        return 0x80000000u;
    unsigned int value = 0;
    if (cudaDeviceSynchronize() != cudaSuccess)
        return 0x80000000u;
    if (cudaMemcpy(&value, st->status, sizeof(value), cudaMemcpyDeviceToHost) != cudaSuccess)
        return 0x80000000u;
    if (value != 0)
        cudaMemset(st->status, 0, sizeof(value));
    return value;
}

#ifdef FLASHLLM_CTA_TIMES
// Launch-shape builds only: copies the per-CTA stamps (4 per CTA, up to 4096 CTAs) to the host.
int FlashLLM_DebugCtaTimes(unsigned long long* out, int count)
{
    cudaDeviceSynchronize();
    return static_cast<int>(cudaMemcpyFromSymbol(out, flashllm::g_cta_times, sizeof(unsigned long long) * count));
}
#endif

#ifdef FLASHLLM_TRACE
// Timeline builds only: copies the recorded timestamps (kinds x depth) to the host.
int FlashLLM_DebugTrace(long long* out, int count)
{
    cudaDeviceSynchronize();
    return static_cast<int>(cudaMemcpyFromSymbol(out, flashllm::g_trace, sizeof(long long) * count));
}
#endif

unsigned long long FlashLLM_LaunchCount(void)
{
    return g_launches.load(std::memory_order_relaxed);
}

}  // extern "C"
