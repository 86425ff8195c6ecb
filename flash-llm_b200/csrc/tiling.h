// Tile geometry and launch-plan description of the sm_100a SpMM.  Takes the place of the reference's
// compile-time TilingConfig / SparseKernelConfig (csrc/TilingConfig.h:16-64).  The tiled-CSL constants are
// fixed by the data format; everything in SpmmPlan is chosen at run time.
#pragma once
#include <stdint.h>

namespace flashllm {

constexpr int kTileM        = 128;   // rows of A per compressed tile (format constant)
constexpr int kTileK        = 64;    // columns of A per compressed tile (format constant)
constexpr int kVectorWords  = 4;     // words per 16-byte vector; tiles are padded to whole vectors
constexpr int kOffsetsExtra = 2;     // TileOffsets holds T + 2 entries
constexpr int kMaxTileVectors = kTileM * kTileK / kVectorWords;  // a fully dense tile: 2048 vectors (32 KB)
constexpr int kDenseTileBytes = kTileM * kTileK * 2;             // 16 KB decompressed fp16 tile
constexpr int kUmmaK          = 16;                              // K extent of one tcgen05.mma (fp16)

constexpr int kMaxAStages      = 12;
constexpr int kMaxBStages      = 8;
constexpr int kMaxRingSlots    = 64;
constexpr int kMaxClusterK     = 8;   // portable cluster size limit
constexpr int kMaxProducers    = 4;   // warps issuing bulk copies of the compressed stream
constexpr int kMaxScatterWarps = 12;
// warps: [0, producers) copy producers, then one B-tile loader, then the MMA issuer / TMEM owner, then scatter warps
constexpr int kMaxThreads = (kMaxProducers + 2 + kMaxScatterWarps) * 32;

// Status bits written by kernels into the per-device status word.
constexpr unsigned kStatusWaitExpired    = 1u;  // a bounded mbarrier wait ran out
constexpr unsigned kStatusBadTileOffsets = 2u;  // a tile's vector range was negative or above 2048
constexpr unsigned kStatusSmemMisaligned = 16u; // dynamic shared memory did not start on a 1024-byte boundary

// Fields of FlashLLM_SetPlan / FlashLLM_GetPlan, in this order.
enum PlanField {
    kPlanClusterK = 0,    // K parts reduced inside a cluster through distributed shared memory (1..8)
    kPlanWorkspaceK,      // K parts reduced through the caller's workspace
    kPlanAStages,         // decompressed 128x64 tiles in flight
    kPlanBStages,         // B batches in flight
    kPlanBBatch,          // K tiles of B fetched by one TMA instruction
    kPlanRingSlots,       // compressed-stream ring: slots ...
    kPlanChunkVectors,    // ... of this many 16-byte vectors (power of two)
    kPlanScatterWarps,    // warps that decompress tiles, one whole tile per warp at a time (4..12, <= a_stages)
    kPlanProducers,       // warps issuing the bulk copies
    kPlanPath,            // how compressed words reach the scatter warps: kPathRing or kPathDirect
    kPlanReduce,          // who adds workspace parts up: kReduceSecondKernel or kReduceLastCta
    kPlanFieldCount
};

constexpr int kReduceSecondKernel = 1;  // splitk_reduce_f32_kernel after the SpMM kernel
constexpr int kReduceLastCta      = 2;  // inside the SpMM kernel, by the last CTA of each output tile to finish

constexpr int kPathRing   = 1;  // bulk copies into a shared-memory ring (spmm_tcgen05_kernel)
constexpr int kPathDirect = 2;  // global loads into the scatter warps' registers (spmm_tcgen05_direct_kernel)

struct SpmmPlan {
    int path;    // kPathRing or kPathDirect
    int n_tile;  // MMA N: 16, 32, 64 or 128
    int cluster_k;
    int workspace_k;
    int a_stages;
    int b_stages;
    int b_batch;
    int ring_slots;
    int chunk_vectors;
    int scatter_warps;
    int producers;
    int reduce;          // kReduceSecondKernel or kReduceLastCta (meaningful when workspace_k > 1)
    int offsets_staged;  // TileOffsets entries a CTA may stage in shared memory (0 = read them from global memory)
    int smem_bytes;      // dynamic shared memory of the launch
};

}  // namespace flashllm
