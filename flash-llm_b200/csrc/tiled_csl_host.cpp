// Host tiled-CSL encoder and file converter behind the reference's InitSparseMatrixA_API,
// InitSparseMatrixA_API_NoReorder and GenSparseMatrixBinFile (reference csrc/SpMM_API.cu:163-555).
//
// Output is bit-identical to the reference's, but it is computed in closed form and in parallel.  The reference
// deals words out one at a time, always popping the newest word of the fullest of 32 shared-memory-bank buckets
// (lowest bucket index on ties, csrc/SpMM_API.cu:145-156,299-320).  That pop order is a level-order walk: with
// bucket sizes c[0..31], it visits height h = max(c) down to 1 and, within a height, every bucket k with c[k] >= h
// in increasing k.  So the pick number of the word at height h of bucket k is
//     q = sum_k' max(0, c[k'] - h)  +  #{k' < k : c[k'] >= h},
// and the reference's two lane-queue passes (tail first, then main, each drained newest-first, :299-346) turn q
// into a fixed output position.  No simulation of the greedy loop is needed.
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>

#include <atomic>
#include <fstream>
#include <thread>
#include <vector>

#include "tiled_csl_host.h"
#include "tiling.h"

namespace flashllm {

// The reference keeps a cell when fabs(float(v)) > 0 (csrc/SpMM_API.cu:184): finite non-zeros and infinities
// pass, +-0 and NaN do not.
static inline bool keeps(uint16_t h)
{
    const uint16_t a = h & 0x7FFFu;
    return a != 0 && a <= 0x7C00u;
}

static inline uint32_t pack(uint16_t value, int loc)
{
    return static_cast<uint32_t>(value) | (static_cast<uint32_t>(loc) << 16);
}

static int count_tile(const uint16_t* tile, size_t ld)
{
    int n = 0;
    for (int m = 0; m < kTileM; ++m) {
        const uint16_t* row = tile + m * ld;
        for (int k = 0; k < kTileK; ++k)
            n += keeps(row[k]) ? 1 : 0;
    }
    return n;
}

// Position, inside a tile of `vectors` 16-byte vectors, of the q-th word the reference's greedy deal picks.
static inline int position_of_pick(int q, int vectors)
{
    const int repeat = vectors / 32, remain = vectors % 32;
    if (q < 4 * remain) {  // tail: lane b = q % remain receives its words in pick order and emits them reversed
        const int v = q / remain, b = q % remain;
        return repeat * 128 + b * 4 + (3 - v);
    }
    const int qm   = q - 4 * remain;
    const int push = qm / 32, b = qm % 32;
    const int w    = 4 * repeat - 1 - push;  // lane queues are drained newest-first
    return (w / 4) * 128 + b * 4 + (w % 4);
}

static void pack_tile_reordered(const uint16_t* tile, size_t ld, uint32_t* dst, int words)
{
    constexpr int kCap = kTileM * kTileK / 32 + kVectorWords;
    static thread_local uint32_t items[32][kCap];
    int count[32], zero_pos[32];
    for (int k = 0; k < 32; ++k) {
        count[k]    = 0;
        zero_pos[k] = -1;
    }
    int nnz = 0;
    for (int m = 0; m < kTileM; ++m) {
        const uint16_t* row = tile + m * ld;
        const int       x   = (m & 7) << 3;
        for (int n = 0; n < kTileK; ++n) {
            const int      colp = n ^ x;
            const int      bank = colp >> 1;
            const int      loc  = m * kTileK + colp;
            const uint16_t v    = row[n];
            if (keeps(v)) {
                items[bank][count[bank]++] = pack(v, loc);
                ++nnz;
            }
            else if (zero_pos[bank] < 0) {
                zero_pos[bank] = loc;
            }
        }
    }
    for (int p = nnz; p < words; ++p) {  // padding words go, one at a time, to the emptiest bucket (:274-287)
        int best = 0;
        for (int k = 1; k < 32; ++k)
            if (count[k] < count[best])
                best = k;
        items[best][count[best]++] = pack(0, zero_pos[best]);
    }
    int top = 0;
    for (int k = 0; k < 32; ++k)
        top = count[k] > top ? count[k] : top;
    const int vectors = words / kVectorWords;
    int       q       = 0;
    for (int h = top; h >= 1; --h)
        for (int k = 0; k < 32; ++k)
            if (count[k] >= h)
                dst[position_of_pick(q++, vectors)] = items[k][h - 1];
}

static void pack_tile_scan_order(const uint16_t* tile, size_t ld, uint32_t* dst, int words, int nnz)
{
    int pads = words - nnz, w = 0;
    for (int m = 0; m < kTileM; ++m) {
        const uint16_t* row = tile + m * ld;
        const int       x   = (m & 7) << 3;
        for (int n = 0; n < kTileK; ++n) {
            const uint16_t v = row[n];
            if (keeps(v))
                dst[w++] = pack(v, m * kTileK + (n ^ x));
            else if (pads > 0) {  // the first cells that test as zero become the padding, bits kept (:456-472)
                --pads;
                dst[w++] = pack(v, m * kTileK + (n ^ x));
            }
        }
    }
}

template<typename F>
static void parallel_for_tiles(int tiles, F&& body)
{
    unsigned hw = std::thread::hardware_concurrency();
    if (hw == 0)
        hw = 1;
    const char* env = getenv("FLASHLLM_ENCODER_THREADS");
    if (env && atoi(env) > 0)
        hw = static_cast<unsigned>(atoi(env));
    const int workers = tiles < 64 ? 1 : static_cast<int>(hw);
    if (workers <= 1) {
        for (int t = 0; t < tiles; ++t)
            body(t);
        return;
    }
    std::atomic<int>         next{0};
    std::vector<std::thread> pool;
    for (int w = 0; w < workers; ++w)
        pool.emplace_back([&]() {
            for (;;) {
                const int begin = next.fetch_add(16);
                if (begin >= tiles)
                    return;
                const int end = begin + 16 < tiles ? begin + 16 : tiles;
                for (int t = begin; t < end; ++t)
                    body(t);
            }
        });
    for (auto& th : pool)
        th.join();
}

int encode_tiled_csl_host(const uint16_t* A, int M, int K, bool reorder, uint32_t** Compressed_A, int** TileOffsets)
{
    if (A == nullptr || Compressed_A == nullptr || TileOffsets == nullptr || M <= 0 || K <= 0 || M % kTileM != 0
        || K % kTileK != 0)
        return -1;
    const int    rows = M / kTileM, cols = K / kTileK;
    const int    T  = rows * cols;
    const size_t ld = static_cast<size_t>(K);
    int*         offs = static_cast<int*>(malloc(static_cast<size_t>(T + kOffsetsExtra) * sizeof(int)));
    if (!offs)
        return -2;
    std::vector<int> nnz_of(T);
    parallel_for_tiles(T, [&](int t) {
        nnz_of[t] = count_tile(A + static_cast<size_t>(t / cols) * kTileM * ld + static_cast<size_t>(t % cols) * kTileK, ld);
    });
    long long total_vectors = 0;
    offs[0]                 = 0;
    for (int t = 0; t < T; ++t) {
        total_vectors += (nnz_of[t] + kVectorWords - 1) / kVectorWords;
        if (total_vectors > 0x7FFFFFFFll) {
            free(offs);
            return -3;  // the format's int offsets cannot address this many vectors
        }
        offs[t + 1] = static_cast<int>(total_vectors);
    }
    offs[T + 1] = offs[T];
    const size_t words = static_cast<size_t>(total_vectors) * kVectorWords;
    uint32_t*    out   = static_cast<uint32_t*>(malloc((words ? words : 1) * sizeof(uint32_t)));
    if (!out) {
        free(offs);
        return -2;
    }
    parallel_for_tiles(T, [&](int t) {
        const uint16_t* tile = A + static_cast<size_t>(t / cols) * kTileM * ld + static_cast<size_t>(t % cols) * kTileK;
        uint32_t*       dst  = out + static_cast<size_t>(offs[t]) * kVectorWords;
        const int       len  = (offs[t + 1] - offs[t]) * kVectorWords;
        if (reorder)
            pack_tile_reordered(tile, ld, dst, len);
        else
            pack_tile_scan_order(tile, ld, dst, len, nnz_of[t]);
    });
    *Compressed_A = out;
    *TileOffsets  = offs;
    return T + kOffsetsExtra;
}

}  // namespace flashllm
