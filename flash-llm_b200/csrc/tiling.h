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

constexpr int kMaxAStages   = 8;
constexpr int kMaxBStages   = 8;
constexpr int kMaxRingSlots = 32;
constexpr int kMaxClusterK  = 8;    // portable cluster size limit
constexpr int kControlWarps = 2;    // warp 0: copy producer, warp 1: MMA issuer + TMEM owner
constexpr int kMaxScatterWarps = 8;
constexpr int kMaxThreads   = (kControlWarps + kMaxScatterWarps) * 32;

// Status bits written by kernels into the per-device status word.
constexpr unsigned kStatusWaitExpired      = 1u;  // a bounded mbarrier wait ran out
constexpr unsigned kStatusBadTileOffsets   = 2u;  // a tile's vector range was negative or above 2048

struct SpmmPlan {
    int n_tile;         // MMA N: 16, 32, 64 or 128
    int cluster_k;      // K parts reduced inside a cluster through distributed shared memory
    int workspace_k;    // K parts reduced through the caller's fp16 workspace
    int a_stages;       // decompressed 128x64 tiles in flight
    int b_stages;       // B tiles in flight
    int ring_slots;     // compressed-stream ring: slots ...
    int chunk_vectors;  // ... of this many 16-byte vectors (power of two)
    int scatter_warps;  // 4 or 8
    int offsets_staged; // TileOffsets entries a CTA may stage in shared memory (0 = read them from global memory)
    int smem_bytes;     // dynamic shared memory of the launch
};

}  // namespace flashllm
