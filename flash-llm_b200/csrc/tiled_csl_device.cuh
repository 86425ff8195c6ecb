// Device tiled-CSL encoder: dense fp16 A in HBM -> TileOffsets and packed words, bit-identical to the host encoder
// and therefore to the reference's InitSparseMatrixA_API / _NoReorder (reference csrc/SpMM_API.cu:163-489).
//
// One warp encodes one 128x64 tile.  For the reordered format lane k owns shared-memory bank k of the decompressed
// tile: the two cells (r, 2k ^ ((r&7)<<3)) and the one after it in every row r, which is exactly the reference's
// bucket k in its row-major scan order (:248-271).  The reference's greedy deal (always pop the newest word of the
// fullest bucket, :299-320) is a level-order walk over bucket heights, so the word at height h of bucket k is pick
//     q = sum_k' max(0, c[k'] - h) + #{k' < k : c[k'] >= h}
// and the two lane-queue passes (:323-346) map q to a fixed slot.  The per-height terms are tabulated once per tile
// in shared memory; every word is then placed independently.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "tiling.h"

namespace flashllm {

constexpr unsigned kStatusOffsetsOverflow  = 4u;  // more 16-byte vectors than an int can count
constexpr unsigned kStatusOffsetsMismatch  = 8u;  // TileOffsets do not match the matrix being packed

constexpr int kEncodeWarps   = 8;
constexpr int kHeightEntries = kTileM * kTileK / 32 + kVectorWords + 1;  // bucket heights 0..259

__device__ __forceinline__ bool keeps_cell(uint32_t h16)
{
    const uint32_t a = h16 & 0x7FFFu;  // the reference keeps finite non-zeros and infinities, drops +-0 and NaN
    return a != 0u && a <= 0x7C00u;
}

__device__ __forceinline__ uint32_t lanemask_lt()
{
    uint32_t m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Output slot of the q-th pick of the reference's deal, inside a tile of `vectors` 16-byte vectors.
__device__ __forceinline__ int slot_of_pick(int q, int vectors)
{
    const int repeat = vectors >> 5, remain = vectors & 31;
    if (q < 4 * remain) {
        const int v = q / remain, b = q - v * remain;
        return repeat * 128 + b * 4 + (3 - v);
    }
    const int qm   = q - 4 * remain;
    const int push = qm >> 5, b = qm & 31;
    const int w    = 4 * repeat - 1 - push;
    return (w >> 2) * 128 + b * 4 + (w & 3);
}

// Step 1a: offs[t + 1] = number of 16-byte vectors of tile t (non-zeros rounded up to a multiple of four).
__global__ void __launch_bounds__(kEncodeWarps * 32)
    csl_count_kernel(const uint16_t* __restrict__ A, int K, int tiles, int k_tiles, int* __restrict__ offs)
{
    const int t    = blockIdx.x * kEncodeWarps + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= tiles)
        return;
    const uint16_t* tile = A + static_cast<size_t>(t / k_tiles) * kTileM * K + static_cast<size_t>(t % k_tiles) * kTileK;
    int             n    = 0;
#pragma unroll 8
    for (int r = 0; r < kTileM; ++r) {
        const uint32_t pair = *reinterpret_cast<const uint32_t*>(tile + static_cast<size_t>(r) * K + 2 * lane);
        n += (keeps_cell(pair & 0xFFFFu) ? 1 : 0) + (keeps_cell(pair >> 16) ? 1 : 0);
    }
    n = __reduce_add_sync(0xFFFFFFFFu, n);
    if (lane == 0)
        offs[t + 1] = (n + kVectorWords - 1) / kVectorWords;
}

// Step 1b: in-place inclusive scan of offs[1..tiles], offs[0] = 0, offs[tiles + 1] = offs[tiles].  One CTA.
__global__ void __launch_bounds__(1024) csl_scan_kernel(int* __restrict__ offs, int tiles, unsigned int* status)
{
    __shared__ long long part[1024];
    const int            tid   = threadIdx.x;
    const int            chunk = (tiles + 1023) / 1024;
    const int            begin = tid * chunk;
    const int            end   = begin + chunk < tiles ? begin + chunk : tiles;
    long long            sum   = 0;
    for (int i = begin; i < end; ++i)
        sum += offs[i + 1];
    part[tid] = sum;
    __syncthreads();
    for (int d = 1; d < 1024; d <<= 1) {
        const long long add = tid >= d ? part[tid - d] : 0;
        __syncthreads();
        part[tid] += add;
        __syncthreads();
    }
    long long run = part[tid] - sum;
    for (int i = begin; i < end; ++i) {
        run += offs[i + 1];
        offs[i + 1] = static_cast<int>(run);
    }
    if (tid == 1023) {
        if (part[1023] > 0x7FFFFFFFll)
            atomicOr(status, kStatusOffsetsOverflow);
        offs[0] = 0;
    }
    __syncthreads();
    if (tid == 0)
        offs[tiles + 1] = static_cast<int>(part[1023]);
}

// Step 2, reordered format.
__global__ void __launch_bounds__(kEncodeWarps * 32) csl_pack_reorder_kernel(const uint16_t* __restrict__ A,
                                                                             int K,
                                                                             int tiles,
                                                                             int k_tiles,
                                                                             const int* __restrict__ offs,
                                                                             uint32_t* __restrict__ out,
                                                                             unsigned int* status)
{
    __shared__ uint32_t s_mask[kEncodeWarps][kHeightEntries];   // buckets at least this high
    __shared__ uint16_t s_above[kEncodeWarps][kHeightEntries];  // words lying above this height (< 8192 + 3)
    const int w    = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int t    = blockIdx.x * kEncodeWarps + w;
    if (t >= tiles)
        return;
    const uint16_t* tile  = A + static_cast<size_t>(t / k_tiles) * kTileM * K + static_cast<size_t>(t % k_tiles) * kTileK;
    const int       first = offs[t];
    const int       vectors = offs[t + 1] - first;
    const int       words   = vectors * kVectorWords;
    uint32_t*       dst     = out + static_cast<size_t>(first) * kVectorWords;

    // pass 1: bucket sizes and each bucket's first zero cell
    int count = 0, zero_loc = -1;
#pragma unroll 4
    for (int r = 0; r < kTileM; ++r) {
        const int      x    = (r & 7) << 3;
        const int      c0   = (2 * lane) ^ x;  // the bucket's two cells sit at columns c0, c0 + 1
        const uint32_t pair = *reinterpret_cast<const uint32_t*>(tile + static_cast<size_t>(r) * K + c0);
        const bool     k0 = keeps_cell(pair & 0xFFFFu), k1 = keeps_cell(pair >> 16);
        count += (k0 ? 1 : 0) + (k1 ? 1 : 0);
        if (zero_loc < 0 && !(k0 && k1))
            zero_loc = r * kTileK + 2 * lane + (k0 ? 1 : 0);
    }
    const int nnz  = __reduce_add_sync(0xFFFFFFFFu, count);
    const int pads = words - nnz;
    if (pads < 0 || pads >= kVectorWords || vectors < 0 || vectors > kMaxTileVectors) {
        if (lane == 0)
            atomicOr(status, kStatusOffsetsMismatch);
        return;
    }
    // padding words join the emptiest bucket, one at a time, lowest bucket on ties
    int total = count;
    for (int p = 0; p < pads; ++p) {
        const unsigned best = __reduce_min_sync(0xFFFFFFFFu, (static_cast<unsigned>(total) << 5) | lane);
        if ((best & 31u) == static_cast<unsigned>(lane))
            ++total;
    }
    const int top = __reduce_max_sync(0xFFFFFFFFu, total);
    // per-height tables, from the top down
    int running = 0;
    for (int h = top; h >= 1; --h) {
        const uint32_t m = __ballot_sync(0xFFFFFFFFu, total >= h);
        if (lane == 0) {
            s_mask[w][h]  = m;
            s_above[w][h] = static_cast<uint16_t>(running);
        }
        running += __popc(m);
    }
    __syncwarp();
    const uint32_t lower = lanemask_lt();

    // pass 2: place every word
    int h = 0;
#pragma unroll 4
    for (int r = 0; r < kTileM; ++r) {
        const int      x    = (r & 7) << 3;
        const int      c0   = (2 * lane) ^ x;
        const uint32_t pair = *reinterpret_cast<const uint32_t*>(tile + static_cast<size_t>(r) * K + c0);
        const uint32_t v0 = pair & 0xFFFFu, v1 = pair >> 16;
        if (keeps_cell(v0)) {
            ++h;
            const int q             = s_above[w][h] + __popc(s_mask[w][h] & lower);
            dst[slot_of_pick(q, vectors)] = v0 | (static_cast<uint32_t>(r * kTileK + 2 * lane) << 16);
        }
        if (keeps_cell(v1)) {
            ++h;
            const int q             = s_above[w][h] + __popc(s_mask[w][h] & lower);
            dst[slot_of_pick(q, vectors)] = v1 | (static_cast<uint32_t>(r * kTileK + 2 * lane + 1) << 16);
        }
    }
    for (; h < total;) {  // this bucket's padding words: +0.0 at its first zero cell
        ++h;
        const int q                   = s_above[w][h] + __popc(s_mask[w][h] & lower);
        dst[slot_of_pick(q, vectors)] = static_cast<uint32_t>(zero_loc) << 16;
    }
}

// Step 2, scan-order format (reference csrc/SpMM_API.cu:441-476): non-zeros in row-major order, with the first
// `pads` zero-testing cells of the tile kept in place as padding words (their bits preserved).
__global__ void __launch_bounds__(kEncodeWarps * 32) csl_pack_scan_kernel(const uint16_t* __restrict__ A,
                                                                          int K,
                                                                          int tiles,
                                                                          int k_tiles,
                                                                          const int* __restrict__ offs,
                                                                          uint32_t* __restrict__ out,
                                                                          unsigned int* status)
{
    const int lane = threadIdx.x & 31;
    const int t    = blockIdx.x * kEncodeWarps + (threadIdx.x >> 5);
    if (t >= tiles)
        return;
    const uint16_t* tile  = A + static_cast<size_t>(t / k_tiles) * kTileM * K + static_cast<size_t>(t % k_tiles) * kTileK;
    const int       first = offs[t];
    const int       words = (offs[t + 1] - first) * kVectorWords;
    uint32_t*       dst   = out + static_cast<size_t>(first) * kVectorWords;

    int nnz = 0;
#pragma unroll 8
    for (int r = 0; r < kTileM; ++r) {
        const uint32_t pair = *reinterpret_cast<const uint32_t*>(tile + static_cast<size_t>(r) * K + 2 * lane);
        nnz += (keeps_cell(pair & 0xFFFFu) ? 1 : 0) + (keeps_cell(pair >> 16) ? 1 : 0);
    }
    nnz            = __reduce_add_sync(0xFFFFFFFFu, nnz);
    const int pads = words - nnz;
    if (pads < 0 || pads >= kVectorWords) {
        if (lane == 0)
            atomicOr(status, kStatusOffsetsMismatch);
        return;
    }
    const uint32_t lower   = lanemask_lt();
    int            emitted = 0, zeros = 0;
    for (int r = 0; r < kTileM; ++r) {
        const int      x    = (r & 7) << 3;
        const uint32_t pair = *reinterpret_cast<const uint32_t*>(tile + static_cast<size_t>(r) * K + 2 * lane);
        const uint32_t v0 = pair & 0xFFFFu, v1 = pair >> 16;
        const bool     k0 = keeps_cell(v0), k1 = keeps_cell(v1);
        bool           e0 = k0, e1 = k1;
        if (zeros < pads) {  // some padding still to place: rank the zero cells of this row
            const uint32_t z0 = __ballot_sync(0xFFFFFFFFu, !k0), z1 = __ballot_sync(0xFFFFFFFFu, !k1);
            const int      zr = zeros + __popc(z0 & lower) + __popc(z1 & lower);
            e0                = k0 || (zr < pads);
            e1                = k1 || (zr + (k0 ? 0 : 1) < pads);
            zeros += __popc(z0) + __popc(z1);
        }
        const uint32_t b0 = __ballot_sync(0xFFFFFFFFu, e0), b1 = __ballot_sync(0xFFFFFFFFu, e1);
        int            pos = emitted + __popc(b0 & lower) + __popc(b1 & lower);
        if (e0)
            dst[pos++] = v0 | (static_cast<uint32_t>(r * kTileK + ((2 * lane) ^ x)) << 16);
        if (e1)
            dst[pos] = v1 | (static_cast<uint32_t>(r * kTileK + ((2 * lane + 1) ^ x)) << 16);
        emitted += __popc(b0) + __popc(b1);
    }
}

}  // namespace flashllm
