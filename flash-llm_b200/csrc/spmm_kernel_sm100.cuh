// Load-as-Sparse / Compute-as-Dense SpMM for sm_100a.
//
// Does the work of the reference's SpMM_Kernel (csrc/SpMM_Kernel.cuh:179-386) and, for the K parts that live in one
// thread-block cluster, of SplitK_Reduction (csrc/Reduction_Kernel.cuh:24-45), with a different machine mapping:
//
//   * One CTA owns one 128-row tile row of A, one N tile of B and a contiguous range of 64-wide K tiles.  The
//     compressed words of that range are contiguous in Compressed_A, so producer warps stream them as fixed-size
//     chunks with cp.async.bulk into a shared-memory ring, regardless of tile boundaries (the reference loads each
//     tile into registers with LDG.128, SpMM_Kernel.cuh:17-62).  Several warps take turns issuing the chunks: bulk
//     copies issued by one warp complete one after another, copies of different warps overlap.
//   * A loader thread fetches B with TMA, several [N_TILE x 64] K tiles per instruction (3-D box, 128-byte swizzle),
//     replacing the per-tile cp.async loader of MatMulUtilities.cuh:39-75.
//   * Scatter groups (a few warps each) decompress whole tiles independently of one another: zero a dense 128x64
//     fp16 stage, then write each word's value at its 16-bit location (SpMM_Kernel.cuh:114-177 does this from
//     registers with the whole CTA).  The location encoding r*64 + (c ^ ((r&7)<<3)) is exactly the 128-byte-swizzled
//     K-major layout tcgen05.mma reads, so reference-encoded buffers work unchanged.
//   * One thread issues four tcgen05.mma (M=128, N=N_TILE, K=16) per stage in tile order, accumulating fp32 in
//     tensor memory (replaces ldmatrix + mma.sync.m16n8k16, MatMulUtilities.cuh:77-132), and hands ring chunks back
//     to the producers once the tiles that overlap them have been decompressed.
//   * Epilogue: TMEM -> registers -> fp16 C.  With cluster_k > 1 the CTAs of a cluster park their fp32 partial tiles
//     in shared memory and each CTA sums and stores a slice of the output through distributed shared memory.
//
// Every mbarrier wait is bounded: on expiry the CTA raises a status bit, all roles leave their loops, in-flight copies
// are given time to land, TMEM is released and the kernel returns.
#pragma once
#include <cuda_fp16.h>

#include "ptx_sm100.cuh"
#include "tiling.h"

namespace flashllm {

struct SpmmParams {
    const uint4*  compressed;    // tiled-CSL words viewed as 16-byte vectors
    const int*    tile_offsets;  // T + 2 prefix sums, in vectors
    half*         out;           // C (used when workspace_k == 1)
    float*        partial;       // workspace_k fp32 partial matrices [N][M] (used when workspace_k > 1)
    unsigned int* status;        // per-device status word
    int           M, N, K;
    int           k_tiles;  // K / 64
    SpmmPlan      plan;
};

constexpr uint64_t kWaitLimitNs = 200ull * 1000ull * 1000ull;

// Pipeline-analysis builds (never the shipped one) drop one stage of the kernel to see what it costs, as the
// reference does with its own stubs (csrc/SpMM_Kernel.cuh:64-111).  Bits: 1 no zero-fill, 2 no scatter stores,
// 4 no MMA, 8 no ring reads, 16 no scatter-group barrier, 32 no B loads.  Results are wrong with any bit set.
#ifndef FLASHLLM_ABLATE
#define FLASHLLM_ABLATE 0
#endif

// Timeline builds (never the shipped one) record SM-clock timestamps of pipeline events of one CTA.
#ifdef FLASHLLM_TRACE
constexpr int kTraceKinds = 24, kTraceDepth = 256;
__device__ long long g_trace[kTraceKinds * kTraceDepth];
#define FL_TRACE(kind, idx)                                                                                             \
    do {                                                                                                               \
        if (blockIdx.y == FLASHLLM_TRACE && blockIdx.x == 0 && (idx) < kTraceDepth)                                    \
            g_trace[(kind) * kTraceDepth + (idx)] = clock64();                                                         \
    } while (0)
#else
#define FL_TRACE(kind, idx)                                                                                             \
    do {                                                                                                               \
    } while (0)
#endif

// Spins on one mbarrier phase.  Returns false when the CTA has been told to give up, or after kWaitLimitNs,
// in which case it raises the abort flag and the status bit itself.
__device__ __forceinline__ bool
wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int* status)
{
    if (ptx::mbar_test_wait(bar, parity))
        return true;
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
#ifdef FLASHLLM_SUSPENDING_WAIT
        if (ptx::mbar_try_wait(bar, parity))  // lets the hardware park the thread; wakes up later than a probe loop
            return true;
#else
        if (ptx::mbar_test_wait(bar, parity))
            return true;
#endif
#ifdef FLASHLLM_WAIT_SLEEP_NS
        __nanosleep(FLASHLLM_WAIT_SLEEP_NS);
#endif
        if ((it & 1023u) == 0u) {
            if (*abort_flag)
                return false;
            const uint64_t now = ptx::globaltimer_ns();
            if (t0 == 0)
                t0 = now;
            else if (now - t0 > kWaitLimitNs) {
                *abort_flag = 1u;
                atomicOr(status, kStatusWaitExpired);
                return false;
            }
        }
    }
}

// Warp-collective form: lane 0 alone probes the mbarrier and the other lanes take its answer at a warp barrier.
// A probe executed by all 32 lanes costs several hundred cycles (measured: ~380 per already-completed wait), so a
// warp must never wait lane by lane.  The warp barrier orders lane 0's observation of the completed phase before
// the other lanes' later reads of the data it guards.
__device__ __forceinline__ bool
wait_bounded_warp(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int* status)
{
    uint32_t ok = 1;
    if ((threadIdx.x & 31) == 0)
        ok = wait_bounded(bar, parity, abort_flag, status) ? 1u : 0u;
    return __shfl_sync(0xFFFFFFFFu, ok, 0) != 0;
}

// OR-reduction over the threads of a named barrier; every participant receives the same answer.
__device__ __forceinline__ bool barrier_any(uint32_t id, uint32_t threads, bool flag)
{
    uint32_t out;
    asm volatile(
        "{\n"
        ".reg .pred p, q;\n"
        "setp.ne.u32 q, %3, 0;\n"
        "bar.red.or.pred p, %1, %2, q;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(out)
        : "r"(id), "r"(threads), "r"(static_cast<uint32_t>(flag))
        : "memory");
    return out != 0;
}

__device__ __forceinline__ void sts_zero16(uint32_t addr)
{
    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(addr), "r"(0u) : "memory");
}

__device__ __forceinline__ uint4 lds16(uint32_t addr)
{
    uint4 v;
    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}

// smem[stage + 2*loc] = value, for one tiled-CSL word (value in the low half, location in the high half).
// Locations are masked to the 8192 cells of a tile so that a corrupt word cannot leave the stage.
__device__ __forceinline__ void scatter_word(uint32_t stage, uint32_t word)
{
    const uint32_t addr = stage + ((word >> 15) & 0x3FFEu);
    asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"(static_cast<unsigned short>(word & 0xFFFFu)) : "memory");
}

__device__ __forceinline__ void scatter_vector(uint32_t stage, const uint4& w)
{
    scatter_word(stage, w.x);
    scatter_word(stage, w.y);
    scatter_word(stage, w.z);
    scatter_word(stage, w.w);
}

template<int N_TILE>
__global__ void __launch_bounds__(kMaxThreads, 1)
    spmm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    constexpr uint32_t kBSlab    = N_TILE * kTileK * 2;  // one K tile of B in shared memory
    constexpr uint32_t kTmemCols = N_TILE < 32 ? 32 : N_TILE;

    extern __shared__ uint8_t smem_raw[];
    const uint32_t            raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t            base     = (raw_addr + 1023u) & ~1023u;  // swizzled operands need 1024-byte alignment
    uint8_t* const            smem     = smem_raw + (base - raw_addr);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;

    const SpmmPlan& plan       = p.plan;
    const int       a_stages   = plan.a_stages;
    const int       b_stages   = plan.b_stages;
    const int       KB         = plan.b_batch;
    const int       ring_slots = plan.ring_slots;
    const int       CV         = plan.chunk_vectors;
    const int       S          = plan.cluster_k;
    const int       G          = plan.workspace_k;
    const int       P          = plan.producers;
    const int       NG         = plan.scatter_groups;
    const int       GW         = plan.warps_per_group;
    const int       NSW        = NG * GW;
    const int       NTS        = NSW * 32;
    const int       b_warp     = P;      // warp that loads B
    const int       mma_warp   = P + 1;  // warp that issues MMAs and owns TMEM
    const int       first_sw   = P + 2;  // first scatter warp
    const int       cv_shift   = 31 - __clz(CV);

    // ---- shared memory carve-up
    const uint32_t a_base     = base;
    const uint32_t b_base     = a_base + a_stages * kDenseTileBytes;
    const uint32_t ring_base  = b_base + b_stages * KB * kBSlab;
    const uint32_t ring_vecs  = ring_slots * CV;
    const uint32_t bar_base   = ring_base + ring_vecs * 16u;
    const uint32_t ring_full  = bar_base;
    const uint32_t ring_empty = ring_full + 8u * ring_slots;
    const uint32_t a_full     = ring_empty + 8u * ring_slots;
    const uint32_t a_empty    = a_full + 8u * a_stages;
    const uint32_t b_full     = a_empty + 8u * a_stages;
    const uint32_t b_empty    = b_full + 8u * b_stages;
    const uint32_t acc_full   = b_empty + 8u * b_stages;
    const uint32_t misc_off   = (acc_full + 8u) - base;
    volatile uint32_t* const tmem_slot  = reinterpret_cast<volatile uint32_t*>(smem + misc_off);
    volatile uint32_t* const abort_flag = reinterpret_cast<volatile uint32_t*>(smem + misc_off + 4);
    volatile int* const      chunks_released = reinterpret_cast<volatile int*>(smem + misc_off + 8);
    int* const               offs_stage = reinterpret_cast<int*>(smem + misc_off + 16);  // plan.offsets_staged ints

    // ---- work assignment: blockIdx.x = K part inside the cluster, y = tile row, z = (N tile, workspace part)
    const int rank     = blockIdx.x;
    const int tile_row = blockIdx.y;
    const int g        = blockIdx.z % G;
    const int n_idx    = blockIdx.z / G;
    const int parts    = S * G;
    const int part     = g * S + rank;
    const int k_begin  = static_cast<int>(static_cast<long long>(p.k_tiles) * part / parts);
    const int k_end    = static_cast<int>(static_cast<long long>(p.k_tiles) * (part + 1) / parts);
    const int L        = k_end - k_begin;
    const int* const offs_global = p.tile_offsets + static_cast<long long>(tile_row) * p.k_tiles + k_begin;
    const bool       staged      = (L + 1 <= plan.offsets_staged);
    const int* const offs        = staged ? offs_stage : offs_global;  // valid after the set-up barrier

    // ---- set-up
    if (threadIdx.x == 0) {
        // An earlier CTA that gave up leaves the status word set; later CTAs then skip their work.
        const unsigned int status_now = *reinterpret_cast<volatile unsigned int*>(p.status);
        for (int i = 0; i < ring_slots; ++i) {
            ptx::mbar_init(ring_full + 8u * i, 1);
            ptx::mbar_init(ring_empty + 8u * i, 1);
        }
        for (int i = 0; i < a_stages; ++i) {
            ptx::mbar_init(a_full + 8u * i, GW);
            ptx::mbar_init(a_empty + 8u * i, 1);
        }
        for (int i = 0; i < b_stages; ++i) {
            ptx::mbar_init(b_full + 8u * i, 1);
            ptx::mbar_init(b_empty + 8u * i, 1);
        }
        ptx::mbar_init(acc_full, 1);
        *abort_flag      = (status_now != 0u) ? 1u : 0u;
        *chunks_released = 0;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == mma_warp) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish();
    }
    if (staged) {
        // This CTA's slice of TileOffsets is read once, together, instead of one dependent load per tile.
        for (int i = threadIdx.x; i <= L; i += blockDim.x)
            offs_stage[i] = offs_global[i];
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp < P) {
        // ================================================================ producers: compressed stream
        if (lane == 0 && L > 0) {
            const int v_first = offs[0];
            int       nvec    = offs[L] - v_first;
            if (nvec < 0)
                nvec = 0;  // the scatter warps report the malformed offsets
            const int    nchunks = (nvec + CV - 1) >> cv_shift;
            const uint4* src     = p.compressed + v_first;
            int          issued  = 0;
            int          slot    = warp % ring_slots;
            uint32_t     use     = warp / ring_slots;
            for (int c = warp; c < nchunks; c += P) {
                FL_TRACE(11, c);
                if (!wait_bounded(ring_empty + 8u * slot, (use & 1u) ^ 1u, abort_flag, p.status))
                    break;
                FL_TRACE(12, c);
                const int      left  = nvec - (c << cv_shift);
                const uint32_t bytes = static_cast<uint32_t>(left < CV ? left : CV) * 16u;
                const uint32_t bar   = ring_full + 8u * slot;
                ptx::mbar_arrive_expect_tx(bar, bytes);
                ptx::bulk_g2s(ring_base + (static_cast<uint32_t>(slot) << cv_shift) * 16u,
                              src + (static_cast<size_t>(c) << cv_shift), bytes, bar);
                ++issued;
                slot += P;
                while (slot >= ring_slots) {
                    slot -= ring_slots;
                    ++use;
                }
            }
            if (*abort_flag) {
                // Give copies already issued a bounded chance to land before the CTA may exit.
                const uint64_t t_leave = ptx::globaltimer_ns();
                for (int back = 0; back < issued && back * P < ring_slots; ++back) {
                    const int      cc  = warp + (issued - 1 - back) * P;
                    const uint32_t bar = ring_full + 8u * (cc % ring_slots);
                    while (!ptx::mbar_test_wait(bar, (cc / ring_slots) & 1u)
                           && ptx::globaltimer_ns() - t_leave < 2000000ull) {}
                }
            }
        }
    }
    else if (warp == b_warp) {
#ifdef FLASHLLM_TRACE
        if (lane == 1 && L > 0) {  // timeline builds: a monitor thread timestamps the landing of every chunk
            const int nvec_m    = offs[L] - offs[0];
            const int nchunks_m = (nvec_m + CV - 1) >> cv_shift;
            for (int c = 0; c < nchunks_m && c < kTraceDepth; ++c) {
                if (!wait_bounded(ring_full + 8u * (c % ring_slots), static_cast<uint32_t>(c / ring_slots) & 1u,
                                  abort_flag, p.status))
                    break;
                FL_TRACE(13, c);
            }
        }
#endif
        // ================================================================ B loader: KB K tiles per TMA instruction
        if (lane == 0 && L > 0 && !(FLASHLLM_ABLATE & 32)) {
            const int batches = (L + KB - 1) / KB;
            int       bs      = 0;
            uint32_t  use     = 0;
            int       issued  = 0;
            for (int b = 0; b < batches; ++b) {
                if (!wait_bounded(b_empty + 8u * bs, (use & 1u) ^ 1u, abort_flag, p.status))
                    break;
                const uint32_t bar = b_full + 8u * bs;
                ptx::mbar_arrive_expect_tx(bar, KB * kBSlab);
                ptx::tma_load_3d(b_base + bs * KB * kBSlab, &tmap_b, 0, n_idx * N_TILE, k_begin + b * KB, bar);
                ++issued;
                if (++bs == b_stages) {
                    bs = 0;
                    ++use;
                }
            }
            if (*abort_flag) {
                const uint64_t t_leave = ptx::globaltimer_ns();
                for (int back = 1; back <= b_stages && back <= issued; ++back) {
                    const int      bb  = issued - back;
                    const uint32_t bar = b_full + 8u * (bb % b_stages);
                    while (!ptx::mbar_test_wait(bar, (bb / b_stages) & 1u)
                           && ptx::globaltimer_ns() - t_leave < 2000000ull) {}
                }
            }
        }
    }
    else if (warp == mma_warp) {
        // ================================================================ MMA issuer (tile order) + ring release
        if (lane == 0 && L > 0) {
            const uint32_t idesc   = ptx::umma_idesc_f16_f32(kTileM, N_TILE);
            const int      v_first = offs[0];
            int            s = 0, bs = 0, kb = 0;
            uint32_t       a_use = 0, b_use = 0;
            int            released = 0, rel_slot = 0;
            for (int j = 0; j < L; ++j) {
                FL_TRACE(7, j);
                if (!wait_bounded(a_full + 8u * s, a_use & 1u, abort_flag, p.status))
                    break;
                FL_TRACE(8, j);
                // Tile j is decompressed: ring chunks that end at or before its last vector are free again.
                const int done = (offs[j + 1] - v_first) >> cv_shift;
                if (released < done) {
                    while (released < done) {
                        FL_TRACE(14, released);
                        ptx::mbar_arrive(ring_empty + 8u * rel_slot);
                        ++released;
                        if (++rel_slot == ring_slots)
                            rel_slot = 0;
                    }
                    *chunks_released = released;
                }
                if (kb == 0 && !(FLASHLLM_ABLATE & 32) && !wait_bounded(b_full + 8u * bs, b_use & 1u, abort_flag, p.status))
                    break;
                FL_TRACE(9, j);
                ptx::tc_fence_after_sync();
                const uint32_t a_addr = a_base + s * kDenseTileBytes;
                const uint32_t b_addr = b_base + (bs * KB + kb) * kBSlab;
#pragma unroll
                for (int kk = 0; kk < ((FLASHLLM_ABLATE & 4) ? 0 : kTileK / kUmmaK); ++kk) {
                    ptx::umma_f16_ss(tmem_acc,
                                     ptx::umma_desc_kmajor_sw128(a_addr + kk * kUmmaK * 2),
                                     ptx::umma_desc_kmajor_sw128(b_addr + kk * kUmmaK * 2),
                                     idesc,
                                     (j | kk) != 0 ? 1u : 0u);
                }
                ptx::umma_commit(a_empty + 8u * s);
                FL_TRACE(10, j);
                if (++s == a_stages) {
                    s = 0;
                    ++a_use;
                }
                if (++kb == KB || j == L - 1) {
                    ptx::umma_commit(b_empty + 8u * bs);
                    kb = 0;
                    if (++bs == b_stages) {
                        bs = 0;
                        ++b_use;
                    }
                }
            }
            ptx::umma_commit(acc_full);
        }
    }
    else {
        // ================================================================ scatter groups: one whole tile at a time
        const int sw   = warp - first_sw;  // scatter warp index
        const int grp  = sw / GW;
        const int gtid = (sw % GW) * 32 + lane;
        const int GT   = GW * 32;
        if (L > 0) {
            const int v_first = offs[0];
            // Stage and ring-slot indices advance by repeated subtraction: a runtime division costs the warp more than
            // a hundred cycles of dependent latency, several times per tile.
            int      s        = grp % a_stages;  // stage of tile j
            uint32_t a_use    = static_cast<uint32_t>(grp / a_stages);
            int      cur_c    = 0;               // a chunk index at or before this tile's first chunk ...
            int      cur_slot = 0;               // ... and its ring slot and use count
            uint32_t cur_use  = 0;
            for (int j = grp; j < L; j += NG, s += NG) {
                if (s >= a_stages) {  // a_stages >= NG: one step is enough
                    s -= a_stages;
                    ++a_use;
                }
                const int      vb    = offs[j] - v_first;
                const int      ve    = offs[j + 1] - v_first;
                const uint32_t stage = a_base + s * kDenseTileBytes;
                const bool     bad   = (ve < vb) || (ve - vb > kMaxTileVectors) || (vb < 0);
                if (bad)
                    atomicOr(p.status, kStatusBadTileOffsets);
                if (gtid == 0)
                    FL_TRACE(0, j);
                bool ok = !bad && wait_bounded_warp(a_empty + 8u * s, (a_use & 1u) ^ 1u, abort_flag, p.status);
                if (gtid == 0)
                    FL_TRACE(1, j);
                if (ok && !(FLASHLLM_ABLATE & 1)) {
                    for (uint32_t off = gtid * 16u; off < kDenseTileBytes; off += GT * 16u)
                        sts_zero16(stage + off);
                }
                if (gtid == 0)
                    FL_TRACE(2, j);
                if (ok && ve > vb) {
                    // Only the chunks this tile overlaps: they cannot be recycled before this tile is done.  A parity
                    // wait is only meaningful once the slot's previous occupant has been handed back, so a group that
                    // has run a whole ring ahead of the tile-order release first waits for that.
                    const int c_first = vb >> cv_shift, c_last = (ve - 1) >> cv_shift;
                    while (cur_c < c_first) {
                        ++cur_c;
                        if (++cur_slot == ring_slots) {
                            cur_slot = 0;
                            ++cur_use;
                        }
                    }
                    if (c_last >= ring_slots && lane == 0) {
                        uint64_t t0 = 0;
                        for (uint32_t it = 1; *chunks_released <= c_last - ring_slots; ++it) {
                            if ((it & 255u) == 0u) {
                                const uint64_t now = ptx::globaltimer_ns();
                                if (*abort_flag) {
                                    ok = false;
                                    break;
                                }
                                if (t0 == 0)
                                    t0 = now;
                                else if (now - t0 > kWaitLimitNs) {
                                    *abort_flag = 1u;
                                    atomicOr(p.status, kStatusWaitExpired);
                                    ok = false;
                                    break;
                                }
                            }
                        }
                    }
                    ok = __shfl_sync(0xFFFFFFFFu, ok ? 1u : 0u, 0) != 0;
                    int      w_slot = cur_slot;
                    uint32_t w_use  = cur_use;
                    if (gtid == 0)
                        FL_TRACE(16, j);
                    for (int c = c_first; c <= c_last && ok; ++c) {
                        ok = wait_bounded_warp(ring_full + 8u * w_slot, w_use & 1u, abort_flag, p.status);
                        if (gtid == 0 && c == c_first)
                            FL_TRACE(17, j);
                        if (++w_slot == ring_slots) {
                            w_slot = 0;
                            ++w_use;
                        }
                    }
                }
                if (gtid == 0) {
                    FL_TRACE(3, j);
#ifdef FLASHLLM_TRACE
                    if (blockIdx.y == FLASHLLM_TRACE && blockIdx.x == 0 && j < kTraceDepth)
                        g_trace[15 * kTraceDepth + j] = ve > vb ? ((ve - 1) >> cv_shift) : -1;
#endif
                }
                // Zeroes must be in place before any warp of the group scatters; the same barrier makes giving up
                // unanimous inside the group.
#if (FLASHLLM_ABLATE & 16)
                if (!ok || *abort_flag != 0u)
                    break;
#else
                if (barrier_any(1 + grp, GT, !ok || *abort_flag != 0u)) {
                    if (bad)
                        *abort_flag = 1u;
                    break;
                }
#endif
                if (gtid == 0)
                    FL_TRACE(4, j);
#if !(FLASHLLM_ABLATE & 8)
                int      v   = vb + gtid;
                uint32_t pos = (static_cast<uint32_t>(cur_slot) << cv_shift) + (static_cast<uint32_t>(vb) & (CV - 1)) + gtid;
                if (pos >= ring_vecs)
                    pos -= ring_vecs;  // GT <= CV <= ring_vecs: one step is enough
                // two vectors per trip so that the second load is in flight while the first is being scattered
                for (; v + GT < ve; v += 2 * GT) {
                    uint32_t pos2 = pos + GT;
                    if (pos2 >= ring_vecs)
                        pos2 -= ring_vecs;
                    const uint4 w0 = lds16(ring_base + pos * 16u);
                    const uint4 w1 = lds16(ring_base + pos2 * 16u);
#if (FLASHLLM_ABLATE & 2)
                    if ((w0.x ^ w0.y ^ w1.z ^ w1.w) == 0x9E3779B9u)  // keeps the loads alive; practically never true
                        scatter_word(stage, w0.x);
#else
                    scatter_vector(stage, w0);
                    scatter_vector(stage, w1);
#endif
                    pos = pos2 + GT;
                    if (pos >= ring_vecs)
                        pos -= ring_vecs;
                }
                if (v < ve) {
                    const uint4 w0 = lds16(ring_base + pos * 16u);
#if (FLASHLLM_ABLATE & 2)
                    if ((w0.x ^ w0.y ^ w0.z ^ w0.w) == 0x9E3779B9u)
                        scatter_word(stage, w0.x);
#else
                    scatter_vector(stage, w0);
#endif
                }
#endif
                if (gtid == 0)
                    FL_TRACE(5, j);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(a_full + 8u * s);
                if (gtid == 0)
                    FL_TRACE(6, j);
            }
        }

        // ================================================================ epilogue (same warps)
        bool acc_ok = true;
        if (L > 0)
            acc_ok = wait_bounded_warp(acc_full, 0u, abort_flag, p.status);
        acc_ok = __all_sync(0xFFFFFFFFu, acc_ok && (*abort_flag == 0u));
        ptx::tc_fence_after_sync();

        const int quarter     = warp & 3;  // TMEM lanes this warp may read: 32*quarter ..
        const int per_quarter = NSW / 4;   // warps sharing a lane quarter split the columns
        const int col_share   = (N_TILE / per_quarter) < 8 ? 8 : (N_TILE / per_quarter);
        const int col_begin   = (sw / 4) * col_share;
        const int col_end     = (col_begin + col_share) < N_TILE ? (col_begin + col_share) : N_TILE;
        const int n_valid     = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
        const int row_in_tile = quarter * 32 + lane;
        const size_t tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
        half* const  out_tile  = p.out + tile_off;
        float* const part_tile = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
        float* const red       = reinterpret_cast<float*>(smem);  // [N_TILE][128] fp32, over the idle A stages

        for (int c0 = col_begin; c0 < col_end; c0 += 8) {
            uint32_t r[8];
            if (L > 0) {
                ptx::tmem_ld_x8(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, r);
                ptx::tmem_wait_ld();
            }
            else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    r[i] = 0u;
            }
            if (S == 1) {
                if (acc_ok) {
#pragma unroll
                    for (int i = 0; i < 8; ++i)
                        if (c0 + i < n_valid) {
                            const size_t at = static_cast<size_t>(c0 + i) * p.M + row_in_tile;
                            if (part_tile)
                                part_tile[at] = __uint_as_float(r[i]);
                            else
                                out_tile[at] = __float2half_rn(__uint_as_float(r[i]));
                        }
                }
            }
            else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    red[(c0 + i) * kTileM + row_in_tile] = __uint_as_float(r[i]);
            }
        }
    }

    // ================================================================ cluster reduction and tear-down
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (S > 1) {
        __syncwarp();
        ptx::cluster_sync_all();  // every CTA's partial tile is parked in its shared memory
        if (warp >= first_sw) {
            const int    tid_s    = threadIdx.x - first_sw * 32;
            const int    n_valid  = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
            const int    total    = N_TILE * kTileM;
            const int    lo       = static_cast<int>(static_cast<long long>(total) * rank / S);
            const int    hi       = static_cast<int>(static_cast<long long>(total) * (rank + 1) / S);
            const bool   store_ok = (*abort_flag == 0u);
            const size_t tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
            half* const  out_tile  = p.out + tile_off;
            float* const part_tile = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
            for (int e = lo + tid_s; e < hi; e += NTS) {
                const int n = e / kTileM, m = e % kTileM;
                if (n >= n_valid)
                    break;
                float acc = 0.0f;
                for (int q = 0; q < S; ++q)
                    acc += ptx::ld_dsmem_f32(ptx::map_to_rank(base + static_cast<uint32_t>(e) * 4u, q));
                if (store_ok) {
                    if (part_tile)
                        part_tile[static_cast<size_t>(n) * p.M + m] = acc;
                    else
                        out_tile[static_cast<size_t>(n) * p.M + m] = __float2half_rn(acc);
                }
            }
        }
        __syncwarp();
        ptx::cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
    }
    if (warp == mma_warp) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_acc, kTmemCols);
    }
}

// Sums the fp32 partial matrices this library parks in the caller's workspace when workspace_k > 1 and rounds once:
// C[i] = fp16(sum_s ws[s*count + i]); four outputs per thread.
__global__ void splitk_reduce_f32_kernel(half* __restrict__ C, const float* __restrict__ ws, long long count, int parts)
{
    const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i4 >= count)
        return;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < parts; ++s) {
        const float4 v = *reinterpret_cast<const float4*>(ws + static_cast<long long>(s) * count + i4);
        acc.x += v.x;
        acc.y += v.y;
        acc.z += v.z;
        acc.w += v.w;
    }
    uint2    o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
    oh[0]       = __floats2half2_rn(acc.x, acc.y);
    oh[1]       = __floats2half2_rn(acc.z, acc.w);
    *reinterpret_cast<uint2*>(C + i4) = o;
}

// The reference's reduction semantics, kept as an entry point of its own (reference csrc/Reduction_Kernel.cuh:24-45):
// C[i] = fp16(sum_s float(ws[s*count + i])) over fp16 partial matrices; eight outputs per thread, 16-byte accesses.
__global__ void splitk_reduce_kernel(half* __restrict__ C, const half* __restrict__ ws, long long count, int parts)
{
    const long long i8 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 8;
    if (i8 >= count)
        return;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i)
        acc[i] = 0.0f;
    for (int s = 0; s < parts; ++s) {
        const uint4   v = *reinterpret_cast<const uint4*>(ws + static_cast<long long>(s) * count + i8);
        const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const float2 f = __half22float2(h[i]);
            acc[2 * i] += f.x;
            acc[2 * i + 1] += f.y;
        }
    }
    uint4    o;
    __half2* oh = reinterpret_cast<__half2*>(&o);
#pragma unroll
    for (int i = 0; i < 4; ++i)
        oh[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
    *reinterpret_cast<uint4*>(C + i8) = o;
}

}  // namespace flashllm
