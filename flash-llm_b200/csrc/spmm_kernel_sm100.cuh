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

constexpr int kMaxPushWorld = 8;  // GPUs of one NVSwitch box (fused all-reduce)

struct SpmmParams {
    const uint4*  compressed;    // tiled-CSL words viewed as 16-byte vectors
    const int*    tile_offsets;  // T + 2 prefix sums, in vectors
    half*         out;           // C (used when workspace_k == 1)
    float*        partial;       // workspace_k fp32 partial matrices [N][M] (used when workspace_k > 1)
    unsigned int* status;        // per-device status word
    const half*   bias;          // [M] added to every output row before the activation, or nullptr
    int           activation;    // kActNone or kActRelu, applied to the fp32 sum before the one fp16 rounding
    const half*   residual;      // [N][M] like C, added after the activation and before the rounding, or nullptr
    int           M, N, K;
    int           k_tiles;  // K / 64
    SpmmPlan      plan;
    // Fused all-reduce of a row-parallel SpMM (push_world > 0): every finished fp32 value of this GPU's partial product
    // is stored into the receive slot this rank owns on every GPU of the group (its own included) instead of C, and
    // each CTA then raises one flag per GPU; allreduce_sum_kernel on each GPU adds the slots up.
    // Split-K sum without a second kernel (workspace_k > 1 and tile_counters != nullptr): every CTA stores its fp32
    // partial tile, then counts itself in on the tile's counter; the CTA that finds all the others already counted adds
    // the parts up in part order and finishes the output.  Nobody waits.  Counters are zero between launches.
    unsigned int* tile_counters;
    int           push_world;
    unsigned int  push_epoch;                  // value the flags are raised to by this call
    float*        push_slot[kMaxPushWorld];    // [N][M] fp32 slot of this rank in GPU w's receive buffer
    unsigned int* push_flag[kMaxPushWorld];    // this rank's flags in GPU w's receive buffer, one per CTA of the grid
};

constexpr uint64_t kWaitLimitNs = 200ull * 1000ull * 1000ull;
// Word index, counted from a CTA's abort flag, of the flag its B loader sets once it is past griddepcontrol.wait.  With
// launch overlap a CTA may sit behind its predecessor kernel for any length of time; the limit of the bounded waits is
// meant for this CTA's own pipeline, so their clocks start only then.
constexpr int kDepsResolved = 2;

// Output epilogue shared by every place that rounds a finished fp32 sum to fp16: optional bias of output feature m,
// optional ReLU, optional residual (element `at` of a matrix laid out like C).  (The reference's callers do this in
// separate passes over fp16 C, third_party/ft.patch ParallelGpt FFN: add_bias_relu after the first FFN GEMM,
// add_bias_residual after the second and after the attention output projection; here it costs one add each and one
// max before the rounding.)
constexpr int kActNone = 0, kActRelu = 1;

__device__ __forceinline__ half finish_output(float acc, const half* bias, int m, int activation, const half* residual,
                                              size_t at)
{
    if (bias != nullptr)
        acc += __half2float(bias[m]);
    if (activation == kActRelu)
        acc = fmaxf(acc, 0.0f);
    if (residual != nullptr)
        acc += __half2float(residual[at]);
    return __float2half_rn(acc);
}

// Pipeline-analysis builds (never the shipped one) drop one stage of the kernel to see what it costs, as the
// reference does with its own stubs (csrc/SpMM_Kernel.cuh:64-111).  Bits: 1 no zero-fill, 2 no scatter stores,
// 8 no ring reads.  Results are wrong with any bit set.
#ifndef FLASHLLM_ABLATE
#define FLASHLLM_ABLATE 0
#endif
#ifndef FLASHLLM_RELAXED_SLEEP_NS
#define FLASHLLM_RELAXED_SLEEP_NS 40
#endif

// Timeline builds (never the shipped one) record SM-clock timestamps of pipeline events of one CTA.
#ifdef FLASHLLM_TRACE
// Timestamps go to shared memory (a global store would sit in front of every later release operation of the thread)
// and are copied out when the CTA finishes.
constexpr int kTraceKinds = 24, kTraceDepth = 96;
__device__ long long g_trace[kTraceKinds * kTraceDepth];
__device__ long long g_trace_origin;
#define FL_TRACE_BASE 40
#define FL_TRACE(kind, idx)                                                                                             \
    do {                                                                                                               \
        if (blockIdx.y == FLASHLLM_TRACE && blockIdx.x == 0 && (idx) >= FL_TRACE_BASE                                  \
            && (idx) < FL_TRACE_BASE + kTraceDepth)                                                                    \
            s_trace[(kind) * kTraceDepth + (idx) - FL_TRACE_BASE] = static_cast<unsigned int>(clock64());             \
    } while (0)
#else
#define FL_TRACE(kind, idx)                                                                                             \
    do {                                                                                                               \
    } while (0)
#endif

// Launch-shape builds (never the shipped one) record four wall-clock stamps per CTA: entry, set-up done, accumulators
// complete, exit.
#ifdef FLASHLLM_CTA_TIMES
__device__ unsigned long long g_cta_times[4 * 4096];
#define FL_CTA_TIME(slot)                                                                                               \
    do {                                                                                                               \
        const unsigned int cta_ = (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x;                      \
        if (cta_ < 4096u)                                                                                              \
            g_cta_times[4u * cta_ + (slot)] = ptx::globaltimer_ns();                                                   \
    } while (0)
#else
#define FL_CTA_TIME(slot)                                                                                               \
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
            if (abort_flag[kDepsResolved] == 0u) {  // still behind the previous kernel of the stream: no clock yet
                t0 = 0;
                continue;
            }
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

// Same wait for the roles that are not on the critical path (scatter groups, copy producers): sleeps between probes so
// that the spinning does not take issue slots from the MMA-issuing thread, whose per-tile loop is the pacing chain.
__device__ __forceinline__ bool
wait_bounded_relaxed(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int* status)
{
    if (ptx::mbar_test_wait(bar, parity))
        return true;
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
        __nanosleep(FLASHLLM_RELAXED_SLEEP_NS);
        if (ptx::mbar_test_wait(bar, parity))
            return true;
        if ((it & 1023u) == 0u) {
            if (*abort_flag)
                return false;
            if (abort_flag[kDepsResolved] == 0u) {  // still behind the previous kernel of the stream: no clock yet
                t0 = 0;
                continue;
            }
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
        ok = wait_bounded_relaxed(bar, parity, abort_flag, status) ? 1u : 0u;
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

// ---------------------------------------------------------------------------------------------------------------
// Pieces shared by the two forms of the kernel
// ---------------------------------------------------------------------------------------------------------------

// This thread's share of the check of a CTA's TileOffsets slice [0, L]: offsets that run backwards or tiles above 2048
// vectors would make the roles of the kernel disagree about who owns which vectors.
__device__ __forceinline__ bool offsets_slice_is_bad(const int* offs_global, int L)
{
    bool bad = false;
    for (int i = threadIdx.x; i < L; i += blockDim.x) {
        const int lo = offs_global[i], hi = offs_global[i + 1];
        bad |= (lo < 0) || (hi < lo) || (hi - lo > kMaxTileVectors);
    }
    return bad;
}

// The B loader thread: `batches` 3-D TMA boxes of KB K tiles of [N_TILE x 64] each into a ring of b_stages buffers.
// B (and, through the MMAs that consume it, every store of the kernel) must come after the kernels before this one in
// the stream; the compressed weights and their offsets are streamed without waiting, which is what the caller promises
// to be safe when it enables launch overlap.
__device__ __forceinline__ void load_b_batches(const CUtensorMap* tmap, int batches, int KB, int b_stages, uint32_t slab_bytes,
                                               uint32_t b_base, uint32_t b_full, uint32_t b_empty, int n_coord, int k_begin,
                                               volatile uint32_t* abort_flag, unsigned int* status)
{
    ptx::grid_dependency_wait();
    abort_flag[kDepsResolved] = 1u;
    int      bs     = 0;
    uint32_t use    = 0;
    int      issued = 0;
    for (int b = 0; b < batches; ++b) {
        if (!wait_bounded_relaxed(b_empty + 8u * bs, (use & 1u) ^ 1u, abort_flag, status))
            break;
        const uint32_t bar = b_full + 8u * bs;
        ptx::mbar_arrive_expect_tx(bar, KB * slab_bytes);
        ptx::tma_load_3d(b_base + bs * KB * slab_bytes, tmap, 0, n_coord, k_begin + b * KB, bar);
        ++issued;
        if (++bs == b_stages) {
            bs = 0;
            ++use;
        }
    }
    if (*abort_flag) {
        // Give copies already issued a bounded chance to land before the CTA may exit.
        const uint64_t t_leave = ptx::globaltimer_ns();
        for (int back = 1; back <= b_stages && back <= issued; ++back) {
            const int      bb  = issued - back;
            const uint32_t bar = b_full + 8u * (bb % b_stages);
            while (!ptx::mbar_test_wait(bar, (bb / b_stages) & 1u) && ptx::globaltimer_ns() - t_leave < 2000000ull) {}
        }
    }
}

// Epilogue of one scatter warp: its share of the accumulator columns from tensor memory (lane quarter `quarter`; the
// first 4 * per_quarter scatter warps split the N_TILE columns, the others idle), summed over the `accumulators`
// accumulators that hold tiles (they lie `acc_stride` columns apart; 0 of them = an empty K range, output 0), then
// stored as fp16 C, as an fp32 partial tile in the workspace, or parked in shared memory (`red`, [N_TILE][128] fp32
// over the idle A stages) for the cluster sum.
template<int N_TILE>
__device__ __forceinline__ void accumulators_to_output(const SpmmParams& p, uint32_t tmem_acc, int accumulators, int acc_stride,
                                                       int quarter, int lane, int sw, int per_quarter, int S, int G, int g,
                                                       int n_idx, int tile_row, bool acc_ok, float* red)
{
    const int col_share   = (N_TILE / per_quarter) < 8 ? 8 : (N_TILE / per_quarter);
    const int col_begin   = sw < 4 * per_quarter ? (sw / 4) * col_share : N_TILE;
    const int col_end     = (col_begin + col_share) < N_TILE ? (col_begin + col_share) : N_TILE;
    const int n_valid     = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
    const int row_in_tile = quarter * 32 + lane;
    const size_t tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
    half* const  out_tile  = p.out + tile_off;
    float* const part_tile = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
    for (int c0 = col_begin; c0 < col_end; c0 += 8) {
        float r[8];
#pragma unroll
        for (int i = 0; i < 8; ++i)
            r[i] = 0.0f;
        if (accumulators == 2) {  // the two loads go out together and are waited for once
            uint32_t t0[8], t1[8];
            ptx::tmem_ld_x8(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + c0, t0);
            ptx::tmem_ld_x8(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + acc_stride + c0, t1);
            ptx::tmem_wait_ld();
#pragma unroll
            for (int i = 0; i < 8; ++i)
                r[i] = __uint_as_float(t0[i]) + __uint_as_float(t1[i]);
        }
        else {
            for (int a = 0; a < accumulators; ++a) {
                uint32_t t[8];
                ptx::tmem_ld_x8(tmem_acc + (static_cast<uint32_t>(quarter * 32) << 16) + a * acc_stride + c0, t);
                ptx::tmem_wait_ld();
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    r[i] += __uint_as_float(t[i]);
            }
        }
        if (S == 1) {
            if (acc_ok) {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (c0 + i < n_valid) {
                        const size_t at = static_cast<size_t>(c0 + i) * p.M + row_in_tile;
                        if (part_tile)
                            part_tile[at] = r[i];
                        else if (p.push_world > 0) {
                            for (int w = 0; w < p.push_world; ++w)
                                p.push_slot[w][tile_off + at] = r[i];
                        }
                        else
                            out_tile[at] = finish_output(r[i], p.bias, tile_row * kTileM + row_in_tile, p.activation, p.residual,
                                                         tile_off + at);
                    }
            }
        }
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                red[(c0 + i) * kTileM + row_in_tile] = r[i];
        }
    }
    if (S == 1 && part_tile != nullptr && p.tile_counters != nullptr)
        __threadfence();  // this thread's partial sums are visible device-wide before the CTA counts itself in
}

// Between the two cluster barriers: every CTA of the cluster has parked its fp32 partial tile [N_TILE][128] at `base`
// of its shared memory; CTA `rank` sums and stores its 1/S share of the tile through distributed shared memory, four
// neighbouring rows per thread.  The S remote loads of a thread are issued together and added in rank order.
template<int N_TILE>
__device__ __forceinline__ void cluster_reduce_store(const SpmmParams& p, uint32_t base, int rank, int S, int G, int g, int n_idx,
                                                     int tile_row, int tid, int threads, bool store_ok)
{
    const int    n_valid  = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
    const int    quads    = N_TILE * (kTileM / 4);
    const int    lo       = static_cast<int>(static_cast<long long>(quads) * rank / S);
    const int    hi       = static_cast<int>(static_cast<long long>(quads) * (rank + 1) / S);
    const size_t tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
    float* const part_tile = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
    const bool   wide_out  = (reinterpret_cast<uintptr_t>(p.out) & 7u) == 0;
    uint32_t     peer[kMaxClusterK];
#pragma unroll
    for (int q = 0; q < kMaxClusterK; ++q)
        peer[q] = q < S ? ptx::map_to_rank(base, q) : 0u;
    for (int e = lo + tid; e < hi; e += threads) {
        const int n = e / (kTileM / 4), m = (e % (kTileM / 4)) * 4;
        if (n >= n_valid)
            break;
        float4 v[kMaxClusterK];
#pragma unroll
        for (int q = 0; q < kMaxClusterK; ++q)
            if (q < S)
                v[q] = ptx::ld_dsmem_v4_f32(peer[q] + static_cast<uint32_t>(e) * 16u);
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int q = 0; q < kMaxClusterK; ++q)
            if (q < S) {
                acc.x += v[q].x;
                acc.y += v[q].y;
                acc.z += v[q].z;
                acc.w += v[q].w;
            }
        if (!store_ok)
            continue;
        const size_t at = static_cast<size_t>(n) * p.M + m;
        if (part_tile)
            *reinterpret_cast<float4*>(part_tile + at) = acc;
        else if (p.push_world > 0) {
            for (int w = 0; w < p.push_world; ++w)
                *reinterpret_cast<float4*>(p.push_slot[w] + tile_off + at) = acc;
        }
        else {
            const int row = tile_row * kTileM + m;
            uint2     o;
            half*     oh = reinterpret_cast<half*>(&o);
            oh[0]        = finish_output(acc.x, p.bias, row, p.activation, p.residual, tile_off + at);
            oh[1]        = finish_output(acc.y, p.bias, row + 1, p.activation, p.residual, tile_off + at + 1);
            oh[2]        = finish_output(acc.z, p.bias, row + 2, p.activation, p.residual, tile_off + at + 2);
            oh[3]        = finish_output(acc.w, p.bias, row + 3, p.activation, p.residual, tile_off + at + 3);
            half* const dst = p.out + tile_off + at;
            if (wide_out)
                *reinterpret_cast<uint2*>(dst) = o;
            else {
                dst[0] = oh[0];
                dst[1] = oh[1];
                dst[2] = oh[2];
                dst[3] = oh[3];
            }
        }
    }
    if (part_tile != nullptr && p.tile_counters != nullptr)
        __threadfence();
}

// Fused all-reduce, sending side: called by every thread of a CTA after its last store of partial sums.  The barrier
// orders the CTA's stores before thread 0's system-scope fence, after which flag `index` of this rank is raised on
// every GPU of the group.  Plain peer stores only.
__device__ __forceinline__ void push_raise_flag(const SpmmParams& p, unsigned int index, bool cta_ok)
{
    if (p.push_world <= 0)
        return;
    __syncthreads();
    if (threadIdx.x == 0 && cta_ok) {  // a CTA that gave up raises nothing: the receivers' waits run out and say so
        __threadfence_system();
        for (int w = 0; w < p.push_world; ++w)
            *reinterpret_cast<volatile unsigned int*>(p.push_flag[w] + index) = p.push_epoch;
    }
}

// One flag per CTA of the grid (every CTA stored a piece of the output).
__device__ __forceinline__ void push_raise_flags(const SpmmParams& p, bool cta_ok)
{
    push_raise_flag(p, (blockIdx.z * gridDim.y + blockIdx.y) * gridDim.x + blockIdx.x, cta_ok);
}

// Word, counted from a CTA's abort flag, that tells its threads whether the CTA is the last of its output tile.
constexpr int kLastOfTile = 1;

// Split-K sum inside the SpMM kernel.  Called by every thread of every CTA after a __syncthreads() that follows the
// CTA's stores of its part of the fp32 partial tile (each storing thread has fenced).  The CTA counts itself in on the
// counter of its output tile; the one that completes the count (`arrivals` = CTAs per output tile) adds the
// workspace parts in part order -- so the result does not depend on which CTA came last -- applies the epilogue and
// stores C, or, in a fused all-reduce, stores the sum into every GPU's receive slot and raises the tile's flag.  The
// counter is back at zero when the launch ends.  No CTA waits for another.
template<int N_TILE>
__device__ __forceinline__ void splitk_sum_by_last_cta(const SpmmParams& p, int arrivals, int G, int n_idx, int tile_row,
                                                       volatile uint32_t* abort_flag)
{
    const unsigned int tile_id = static_cast<unsigned int>(n_idx) * gridDim.y + tile_row;
    if (threadIdx.x == 0) {
        // arrivals in the low half of the counter; a CTA that gave up also marks the high half, so that the last one
        // knows the tile's sum is not to be trusted
        const unsigned int mine = *abort_flag == 0u ? 1u : 0x10001u;
        // The counters and the parts may still be in use by the launch before this one on the stream until it has
        // completed; a CTA that did no work has not waited for that yet (for the others this returns at once).
        ptx::grid_dependency_wait();
        __threadfence();
        const unsigned int before = atomicAdd(p.tile_counters + tile_id, mine);
        const bool         last   = (before & 0xFFFFu) + 1u == static_cast<unsigned int>(arrivals);
        if (last)
            atomicExch(p.tile_counters + tile_id, 0u);  // nobody else touches it again in this launch
        abort_flag[kLastOfTile] = last ? (((before + mine) >> 16) != 0u ? 2u : 1u) : 0u;
    }
    __syncthreads();
    const unsigned int role = abort_flag[kLastOfTile];
    if (role == 0u)
        return;
    __threadfence();  // the other CTAs' partial sums, stored before they counted themselves in, are visible from here on
    const int    n_valid  = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
    const size_t tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
    const size_t count    = static_cast<size_t>(p.M) * p.N;
    for (int q = threadIdx.x; q < n_valid * (kTileM / 4); q += blockDim.x) {
        const int    n  = q / (kTileM / 4), m = (q % (kTileM / 4)) * 4;
        const size_t at = tile_off + static_cast<size_t>(n) * p.M + m;
        float4       acc = make_float4(0.f, 0.f, 0.f, 0.f);
        for (int g0 = 0; g0 < G; g0 += 4) {  // four parts' loads in flight at a time, added in part order
            float4 v[4];
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (g0 + j < G)
                    v[j] = __ldcg(reinterpret_cast<const float4*>(p.partial + static_cast<size_t>(g0 + j) * count + at));
#pragma unroll
            for (int j = 0; j < 4; ++j)
                if (g0 + j < G) {
                    acc.x += v[j].x;
                    acc.y += v[j].y;
                    acc.z += v[j].z;
                    acc.w += v[j].w;
                }
        }
        if (p.push_world > 0) {
            for (int w = 0; w < p.push_world; ++w)
                *reinterpret_cast<float4*>(p.push_slot[w] + at) = acc;
        }
        else {
            const int row = tile_row * kTileM + m;
            uint2     o;
            half*     oh = reinterpret_cast<half*>(&o);
            oh[0]        = finish_output(acc.x, p.bias, row, p.activation, p.residual, at);
            oh[1]        = finish_output(acc.y, p.bias, row + 1, p.activation, p.residual, at + 1);
            oh[2]        = finish_output(acc.z, p.bias, row + 2, p.activation, p.residual, at + 2);
            oh[3]        = finish_output(acc.w, p.bias, row + 3, p.activation, p.residual, at + 3);
            *reinterpret_cast<uint2*>(p.out + at) = o;
        }
    }
    push_raise_flag(p, tile_id, role == 1u);  // a tile with a part missing raises nothing: the receivers' waits say so
}

// What every CTA does after its part of the output has left it: the in-kernel split-K sum, or its flag of a fused
// all-reduce whose partial sums went straight to the receive slots.
template<int N_TILE>
__device__ __forceinline__ void finish_tile(const SpmmParams& p, int S, int G, int n_idx, int tile_row,
                                            volatile uint32_t* abort_flag)
{
    if (G > 1 && p.tile_counters != nullptr)
        splitk_sum_by_last_cta<N_TILE>(p, S * G, G, n_idx, tile_row, abort_flag);
    else
        push_raise_flags(p, *abort_flag == 0u);
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

// Zeroes one 16 KB stage with the 32 lanes of a scatter warp, fully unrolled: 32 stores of 16 bytes per lane.
__device__ __forceinline__ void zero_fill_stage(uint32_t stage, int lane)
{
#pragma unroll
    for (int q = 0; q < kDenseTileBytes / (32 * 16); ++q)
        sts_zero16(stage + static_cast<uint32_t>(q * 32 + lane) * 16u);
}

// N_TILE: MMA N (tokens per CTA).  The per-tile paths of every role are latency-bound chains of a few dozen
// instructions: each shared-memory or mbarrier round trip in them costs 30-150 cycles and nothing else runs in that
// thread meanwhile.  Hence straight-line code, probes issued side by side or ahead of time, no runtime divisions,
// and no cross-warp hand-offs other than the mbarriers themselves.
template<int N_TILE>
__global__ void __launch_bounds__(kMaxThreads, 1)
    spmm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    constexpr uint32_t kBSlab    = N_TILE * kTileK * 2;  // one K tile of B in shared memory
    constexpr uint32_t kTmemCols = N_TILE < 32 ? 32 : N_TILE;

#ifdef FLASHLLM_TRACE
    __shared__ unsigned int s_trace[kTraceKinds * kTraceDepth];
    for (int i = threadIdx.x; i < kTraceKinds * kTraceDepth; i += blockDim.x)
        s_trace[i] = 0;
#endif
    extern __shared__ __align__(1024) uint8_t smem_raw[];
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
    const int       NSW        = plan.scatter_warps;  // each scatter warp decompresses whole tiles on its own
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
    volatile int* const      tiles_scattered = reinterpret_cast<volatile int*>(smem + misc_off + 8);
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

    if (raw_addr != base) {  // the launch did not honour the 1024-byte alignment: nothing below would be valid
        if (threadIdx.x == 0)
            atomicOr(p.status, kStatusSmemMisaligned);
        return;
    }

    // ---- set-up
    if (threadIdx.x == 0) {
        for (int i = 0; i < ring_slots; ++i) {
            ptx::mbar_init(ring_full + 8u * i, 1);
            // a slot is free again once every one of its CV vectors has been consumed: the warps that consume them
            // arrive with the number of vectors they took, in whatever order the tiles finish
            ptx::mbar_init(ring_empty + 8u * i, CV);
        }
        for (int i = 0; i < a_stages; ++i) {
            ptx::mbar_init(a_full + 8u * i, 1);
            ptx::mbar_init(a_empty + 8u * i, 1);
        }
        for (int i = 0; i < b_stages; ++i) {
            ptx::mbar_init(b_full + 8u * i, 1);
            ptx::mbar_init(b_empty + 8u * i, 1);
        }
        ptx::mbar_init(acc_full, 1);
        abort_flag[0]             = 0u;  // a launch never inherits a give-up from an earlier one: the status word only reports
        abort_flag[kDepsResolved] = 0u;
        *tiles_scattered          = 0;
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
    // Offsets that run backwards, or tiles above 2048 vectors, would make the roles below disagree about who owns
    // which vectors; the whole slice is checked before any of them starts.
    bool bad_slice = offsets_slice_is_bad(offs_global, L);
    ptx::tc_fence_before_sync();
    bad_slice = __syncthreads_or(bad_slice ? 1 : 0) != 0;
    ptx::tc_fence_after_sync();
    const bool go = !bad_slice && (*abort_flag == 0u);  // false: every role skips its work and nothing is stored
    if (bad_slice && threadIdx.x == 0) {
        atomicOr(p.status, kStatusBadTileOffsets);
        *abort_flag = 1u;
    }
    const uint32_t tmem_acc = *tmem_slot;
    // A following kernel of this library may start its own set-up and weight streaming while this grid drains; it
    // waits (below, in its B loader) before it touches anything this grid or its predecessors produce.
    if (threadIdx.x == 0)
        ptx::grid_launch_dependents();

    if (warp < P) {
        // ================================================================ producers: compressed stream
        if (lane == 0 && L > 0 && go) {
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
                if (!wait_bounded_relaxed(ring_empty + 8u * slot, (use & 1u) ^ 1u, abort_flag, p.status))
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
        // ================================================================ B loader: KB K tiles per TMA instruction
        if (lane == 0 && L > 0 && go && !(FLASHLLM_ABLATE & 32)) {
            load_b_batches(&tmap_b, (L + KB - 1) / KB, KB, b_stages, kBSlab, b_base, b_full, b_empty, n_idx * N_TILE, k_begin,
                           abort_flag, p.status);
        }
    }
    else if (warp == mma_warp) {
        // ================================================================ MMA issuer (tile order)
        // Per tile: four MMAs, the commit that hands the stage back, and a probe of the next tile's barriers issued
        // ahead of the MMAs so that its round trip is hidden behind them.
        if (lane == 0 && L > 0 && go) {
            const uint32_t idesc   = ptx::umma_idesc_f16_f32(kTileM, N_TILE);
            const uint64_t a_desc0 = ptx::umma_desc_kmajor_sw128(a_base);
            const uint64_t b_desc0 = ptx::umma_desc_kmajor_sw128(b_base);
            int            s = 0, bs = 0, kb = 0;
            uint32_t       a_par = 0, b_par = 0;
            bool           ready = false;
            for (int j = 0; j < L; ++j) {
                FL_TRACE(7, j);
                if (!ready) {
                    if (!wait_bounded(a_full + 8u * s, a_par, abort_flag, p.status))
                        break;
                    if (kb == 0 && !wait_bounded(b_full + 8u * bs, b_par, abort_flag, p.status))
                        break;
                }
                FL_TRACE(9, j);
                int      s_n = s + 1, kb_n = kb + 1, bs_n = bs;
                uint32_t a_par_n = a_par, b_par_n = b_par;
                if (s_n == a_stages) {
                    s_n = 0;
                    a_par_n ^= 1u;
                }
                if (kb_n == KB) {
                    kb_n = 0;
                    if (++bs_n == b_stages) {
                        bs_n = 0;
                        b_par_n ^= 1u;
                    }
                }
                const bool has_next = j + 1 < L;
                ptx::tc_fence_after_sync();
                ready = ptx::umma_tile_commit_probe(
                    tmem_acc, a_desc0 + static_cast<uint32_t>(s * (kDenseTileBytes >> 4)),
                    b_desc0 + static_cast<uint32_t>((bs * KB + kb) * (kBSlab >> 4)), idesc, j != 0 ? 1u : 0u, a_empty + 8u * s,
                    b_empty + 8u * bs, (kb_n == 0 || !has_next) ? 1u : 0u, a_full + 8u * s_n, a_par_n, b_full + 8u * bs_n, b_par_n,
                    has_next ? 1u : 0u, (has_next && kb_n == 0) ? 1u : 0u);
                FL_TRACE(10, j);
                *tiles_scattered = j + 1;
                s     = s_n;
                kb    = kb_n;
                bs    = bs_n;
                a_par = a_par_n;
                b_par = b_par_n;
                FL_TRACE(19, j);
            }
            ptx::umma_commit(acc_full);
        }
    }
    else {
        // ================================================================ scatter warps: one whole tile at a time
        const int sw = warp - first_sw;  // scatter warp index
        if (L > 0 && go) {
            const int v_first = offs[0];
            // Stage and ring-slot indices advance by repeated subtraction: a runtime division costs the warp more than
            // a hundred cycles of dependent latency, several times per tile.
            int      s        = sw % a_stages;  // stage of tile j
            uint32_t a_use    = static_cast<uint32_t>(sw / a_stages);
            int      cur_c    = 0;              // a chunk index at or before this tile's first chunk ...
            int      cur_slot = 0;              // ... and its ring slot and use count
            uint32_t cur_use  = 0;
            int      vb_next  = sw < L ? offs[sw] - v_first : 0;  // offsets are fetched one tile ahead of their use
            int      ve_next  = sw < L ? offs[sw + 1] - v_first : 0;
            for (int j = sw; j < L; j += NSW, s += NSW) {
                if (s >= a_stages) {  // a_stages >= NSW: one step is enough
                    s -= a_stages;
                    ++a_use;
                }
                const int vb = vb_next, ve = ve_next;
                if (j + NSW < L) {
                    vb_next = offs[j + NSW] - v_first;
                    ve_next = offs[j + NSW + 1] - v_first;
                }
                // end of the newest tile whose MMA must have finished before this stage was handed back to us
                const int      settled = j >= a_stages ? offs[j - a_stages + 1] - v_first : 0;
                const uint32_t stage   = a_base + s * kDenseTileBytes;
                const bool     bad     = (ve < vb) || (ve - vb > kMaxTileVectors) || (vb < 0);
                if (bad)
                    atomicOr(p.status, kStatusBadTileOffsets);
                if (lane == 0)
                    FL_TRACE(0, j);
                const int c_first = vb >> cv_shift;
                const int n_chunk = ve > vb ? (((ve - 1) >> cv_shift) - c_first + 1) : 0;
                while (cur_c < c_first) {
                    ++cur_c;
                    if (++cur_slot == ring_slots) {
                        cur_slot = 0;
                        ++cur_use;
                    }
                }
                bool ok = !bad;
                // A parity probe of a ring slot means something only once the slot's previous occupant has landed.
                // That is certain when that occupant ends inside tiles whose MMA has already completed (which our
                // stage hand-back proves); otherwise (very dense tiles) wait for the tile counter first.
                const int c_last = c_first + n_chunk - 1;
                if (ok && n_chunk > 0 && c_last >= ring_slots && ((c_last - ring_slots + 1) << cv_shift) > settled) {
                    if (lane == 0) {
                        int need = j;  // last tile that overlaps the previous occupant
                        while (need > 0 && offs[need] - v_first >= ((c_last - ring_slots + 1) << cv_shift))
                            --need;
                        uint64_t t0 = 0;
                        for (uint32_t it = 1; *tiles_scattered <= need; ++it) {
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
                }
                // ---- everything this tile waits for, probed side by side: lane 0 the stage, lanes 1.. the ring chunks
                uint32_t my_slot_bar = 0;  // lanes 1..n_chunk: byte offset of their chunk's barrier pair
                uint32_t my_count    = 0;  // ... and the number of this tile's vectors inside that chunk
                if (ok) {
                    uint32_t my_bar, my_par;
                    bool     mine;
                    if (lane == 0) {
                        my_bar = a_empty + 8u * s;
                        my_par = (a_use & 1u) ^ 1u;
                        mine   = true;
                    }
                    else {
                        int      slot = cur_slot + (lane - 1);
                        uint32_t use  = cur_use;
                        if (slot >= ring_slots) {  // a tile spans at most ring_slots chunks
                            slot -= ring_slots;
                            ++use;
                        }
                        my_slot_bar = 8u * slot;
                        my_bar      = ring_full + my_slot_bar;
                        my_par      = use & 1u;
                        mine        = lane - 1 < n_chunk;
                        if (mine) {
                            const int c  = c_first + lane - 1;
                            const int lo = vb > (c << cv_shift) ? vb : (c << cv_shift);
                            const int hi = ve < ((c + 1) << cv_shift) ? ve : ((c + 1) << cv_shift);
                            my_count     = static_cast<uint32_t>(hi - lo);
                        }
                    }
                    bool ready = !mine || ptx::mbar_test_wait(my_bar, my_par);
                    if (!__all_sync(0xFFFFFFFFu, ready)) {
                        if (mine && !ready)
                            ready = wait_bounded_relaxed(my_bar, my_par, abort_flag, p.status);
                        ok = __all_sync(0xFFFFFFFFu, ready);
                    }
                }
                if (lane == 0)
                    FL_TRACE(3, j);
                if (ok && !(FLASHLLM_ABLATE & 1))
                    zero_fill_stage(stage, lane);
                if (lane == 0)
                    FL_TRACE(2, j);
                // the warp barrier orders the zero stores before the scatter stores of other lanes
                if (__any_sync(0xFFFFFFFFu, !ok)) {
                    if (bad)
                        *abort_flag = 1u;
                    break;
                }
#if !(FLASHLLM_ABLATE & 8)
                int      v   = vb + lane;
                uint32_t pos = (static_cast<uint32_t>(cur_slot) << cv_shift) + (static_cast<uint32_t>(vb) & (CV - 1)) + lane;
                if (pos >= ring_vecs)
                    pos -= ring_vecs;
                // four vectors per trip: the loads are issued together, then their sixteen stores
                for (; v + 96 < ve; v += 128) {
                    uint32_t p1 = pos + 32;
                    if (p1 >= ring_vecs)
                        p1 -= ring_vecs;
                    uint32_t p2 = p1 + 32;
                    if (p2 >= ring_vecs)
                        p2 -= ring_vecs;
                    uint32_t p3 = p2 + 32;
                    if (p3 >= ring_vecs)
                        p3 -= ring_vecs;
                    const uint4 w0 = lds16(ring_base + pos * 16u);
                    const uint4 w1 = lds16(ring_base + p1 * 16u);
                    const uint4 w2 = lds16(ring_base + p2 * 16u);
                    const uint4 w3 = lds16(ring_base + p3 * 16u);
#if (FLASHLLM_ABLATE & 2)
                    if ((w0.x ^ w1.y ^ w2.z ^ w3.w) == 0x9E3779B9u)  // keeps the loads alive; practically never true
                        scatter_word(stage, w0.x);
#else
                    scatter_vector(stage, w0);
                    scatter_vector(stage, w1);
                    scatter_vector(stage, w2);
                    scatter_vector(stage, w3);
#endif
                    pos = p3 + 32;
                    if (pos >= ring_vecs)
                        pos -= ring_vecs;
                }
                for (; v < ve; v += 32) {
                    const uint4 w0 = lds16(ring_base + pos * 16u);
#if (FLASHLLM_ABLATE & 2)
                    if ((w0.x ^ w0.y ^ w0.z ^ w0.w) == 0x9E3779B9u)
                        scatter_word(stage, w0.x);
#else
                    scatter_vector(stage, w0);
#endif
                    pos += 32;
                    if (pos >= ring_vecs)
                        pos -= ring_vecs;
                }
#endif
                if (lane == 0)
                    FL_TRACE(5, j);
                ptx::fence_proxy_async_smem();
                __syncwarp();
                // lane 0 publishes the tile; the lanes that watched a ring chunk hand its vectors back
                if (lane == 0)
                    ptx::mbar_arrive(a_full + 8u * s);
                else if (my_count != 0)
                    ptx::mbar_arrive_count(ring_empty + my_slot_bar, my_count);
                if (lane == 0)
                    FL_TRACE(6, j);
            }
        }

        // ================================================================ epilogue (same warps)
        bool acc_ok = go;
        if (L > 0 && go)
            acc_ok = wait_bounded_warp(acc_full, 0u, abort_flag, p.status);
        acc_ok = __all_sync(0xFFFFFFFFu, acc_ok && (*abort_flag == 0u));
        ptx::tc_fence_after_sync();

        accumulators_to_output<N_TILE>(p, tmem_acc, L > 0 ? 1 : 0, N_TILE, warp & 3, lane, sw, NSW >= 8 ? 2 : 1, S, G, g, n_idx,
                                       tile_row, acc_ok, reinterpret_cast<float*>(smem));
    }

    // ================================================================ cluster reduction and tear-down
    ptx::tc_fence_before_sync();
    __syncthreads();
    if (S > 1) {
        __syncwarp();
        ptx::cluster_sync_all();  // every CTA's partial tile is parked in its shared memory
        if (warp >= first_sw)
            cluster_reduce_store<N_TILE>(p, base, rank, S, G, g, n_idx, tile_row, threadIdx.x - first_sw * 32, NTS,
                                         *abort_flag == 0u);
        __syncwarp();
        ptx::cluster_sync_all();  // nobody leaves while a peer may still read its shared memory
    }
    finish_tile<N_TILE>(p, S, G, n_idx, tile_row, abort_flag);
    if (warp == mma_warp) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_acc, kTmemCols);
    }
#ifdef FLASHLLM_TRACE
    if (blockIdx.y == FLASHLLM_TRACE && blockIdx.x == 0)
        for (int i = threadIdx.x; i < kTraceKinds * kTraceDepth; i += blockDim.x)
            g_trace[i] = s_trace[i];
#endif
}

// Sums the fp32 partial matrices this library parks in the caller's workspace when workspace_k > 1 and rounds once:
// C[i] = fp16(sum_s ws[s*count + i]); four outputs per thread.
__global__ void splitk_reduce_f32_kernel(half* __restrict__ C, const float* __restrict__ ws, long long count, int parts,
                                         const half* __restrict__ bias, int M, int activation,
                                         const half* __restrict__ residual)
{
    ptx::grid_launch_dependents();  // the next SpMM may begin streaming its weights
    ptx::grid_dependency_wait();    // the partial matrices come from the SpMM launched just before
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
    const int m = static_cast<int>(i4 % M);  // C is [N][M] and M is a multiple of 4: the four share a row of C
    uint2     o;
    half*     oh = reinterpret_cast<half*>(&o);
    oh[0]        = finish_output(acc.x, bias, m, activation, residual, static_cast<size_t>(i4));
    oh[1]        = finish_output(acc.y, bias, m + 1, activation, residual, static_cast<size_t>(i4) + 1);
    oh[2]        = finish_output(acc.z, bias, m + 2, activation, residual, static_cast<size_t>(i4) + 2);
    oh[3]        = finish_output(acc.w, bias, m + 3, activation, residual, static_cast<size_t>(i4) + 3);
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

constexpr unsigned kStatusPeerWaitExpired = 32u;  // a GPU of the group did not deliver its partial sums in time

// Fused all-reduce, receiving side: C = fp16(act(sum over the group's GPUs of their fp32 partial products + bias)).
// `slots` holds `world` matrices [N][M] fp32, `slot_stride` floats apart (slot w written by GPU w); `flags` holds, for
// each sender, `flag_stride` words: `flags_per_tile` consecutive ones per output tile (tile index = N tile *
// tile_rows + tile row), one per CTA that stored a piece of the tile (a cluster's CTAs), or one for the tile when the
// last CTA of a tile sent its sum.  A warp covers 128 consecutive outputs = one row segment of ONE output tile, so it
// waits only for that tile's flags: lane l polls flag l % flags_per_tile of sender l / flags_per_tile (at most
// 8 senders x 8 flags, two per lane), for at most `wait_limit_ns`.  A sender raises a flag after the stores it stands
// for.  Slots are added in rank order on every GPU, so all GPUs get the same bits.
// `stream_ordered` != 0: the kernel first waits for everything enqueued before it on its stream (needed when the
// senders are kernels of the same stream on the same GPU: nothing else guarantees that they run at all while this
// one polls).  With 0 the flags are the only dependency: this GPU's sender is the launch right before, all of whose
// CTAs are resident or finished by the time a dependent launch starts, and the other senders run on other GPUs; the
// kernel then neither waits for its predecessor to drain nor for its peer stores to be flushed.
__global__ void allreduce_sum_kernel(half* __restrict__ C, const float* slots, long long slot_stride,
                                     const unsigned int* flags, int flag_stride, unsigned int epoch, int world,
                                     int flags_per_tile, int tile_rows, int n_tile, long long count,
                                     const half* __restrict__ bias, int M, int activation,
                                     const half* __restrict__ residual, unsigned int* status,
                                     unsigned long long wait_limit_ns, int stream_ordered)
{
#ifdef FLASHLLM_CTA_TIMES
#define FL_SUM_TIME(slot)                                                                                               \
    do {                                                                                                               \
        if (threadIdx.x == 0 && (blockIdx.x == 0 || blockIdx.x == gridDim.x - 1))                                      \
            g_cta_times[4u * (4000u + (blockIdx.x == 0 ? 0u : 1u)) + (slot)] = ptx::globaltimer_ns();                  \
    } while (0)
#else
#define FL_SUM_TIME(slot)                                                                                               \
    do {                                                                                                               \
    } while (0)
#endif
    FL_SUM_TIME(0);
    ptx::grid_launch_dependents();
    if (stream_ordered)
        ptx::grid_dependency_wait();
    const long long i4 = (static_cast<long long>(blockIdx.x) * blockDim.x + threadIdx.x) * 4;
    if (i4 - (threadIdx.x & 31) * 4 >= count)  // the whole warp lies past the end (count is a multiple of 128)
        return;
    const int lane = threadIdx.x & 31;
    const int n    = static_cast<int>(i4 / M);
    const int m    = static_cast<int>(i4 % M);
    const int tile = (n / n_tile) * tile_rows + m / kTileM;  // the same for all lanes of the warp
    const int mine = world * flags_per_tile;                  // flags this warp depends on (<= 64)
    bool      ok   = true;
    uint64_t  t0   = 0;
    for (int f = lane; f < mine && ok; f += 32) {
        const unsigned int* flag =
            flags + static_cast<long long>(f / flags_per_tile) * flag_stride + tile * flags_per_tile + f % flags_per_tile;
        for (uint32_t it = 1;; ++it) {
            // the acquire pairs with the sender's release of this flag: once the flag has reached this call's number,
            // the sender's partial sums are visible.  Flags only ever grow (one step per call): "reached" = not
            // behind, also across the 32-bit wrap.
            if (static_cast<int>(ptx::ld_acquire_sys_u32(flag) - epoch) >= 0)
                break;
            __nanosleep(64);
            if ((it & 255u) == 0u) {
                const uint64_t now = ptx::globaltimer_ns();
                if (t0 == 0)
                    t0 = now;
                else if (now - t0 > wait_limit_ns) {
                    ok = false;
                    break;
                }
            }
        }
    }
    FL_SUM_TIME(1);
    ok = __all_sync(0xFFFFFFFFu, ok);  // also orders every lane of the warp after the flags its lanes acquired
    FL_SUM_TIME(2);
    if (!ok) {
        if (lane == 0)
            atomicOr(status, kStatusPeerWaitExpired);
        return;  // nothing is stored for this tile row segment: the caller reads the status word
    }
    float4 v[kMaxPushWorld];
#pragma unroll
    for (int w = 0; w < kMaxPushWorld; ++w)  // all senders' values requested together, added in rank order
        if (w < world)
            v[w] = __ldcg(reinterpret_cast<const float4*>(slots + static_cast<long long>(w) * slot_stride + i4));
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int w = 0; w < kMaxPushWorld; ++w)
        if (w < world) {
            acc.x += v[w].x;
            acc.y += v[w].y;
            acc.z += v[w].z;
            acc.w += v[w].w;
        }
    uint2 o;
    half* oh = reinterpret_cast<half*>(&o);
    oh[0]    = finish_output(acc.x, bias, m, activation, residual, static_cast<size_t>(i4));
    oh[1]    = finish_output(acc.y, bias, m + 1, activation, residual, static_cast<size_t>(i4) + 1);
    oh[2]    = finish_output(acc.z, bias, m + 2, activation, residual, static_cast<size_t>(i4) + 2);
    oh[3]    = finish_output(acc.w, bias, m + 3, activation, residual, static_cast<size_t>(i4) + 3);
    *reinterpret_cast<uint2*>(C + i4) = o;
    FL_SUM_TIME(3);
}

}  // namespace flashllm
