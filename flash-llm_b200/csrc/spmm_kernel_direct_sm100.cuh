// Load-as-Sparse / Compute-as-Dense SpMM for sm_100a, register-streaming form.
//
// Same work, roles of the B loader, MMA issuer and epilogue, K split and bounded waits as spmm_tcgen05_kernel, but
// the compressed words never pass through shared memory as a stream:
//
//   * Every scatter warp owns one 16 KB stage and takes every NSW-th tile of the CTA's K range.  It fetches the words
//     of its NEXT tile straight from global memory into registers (ld.global.nc, 16 bytes per lane and instruction,
//     the reference's LDG.128 scheme, csrc/SpMM_Kernel.cuh:17-62) right after it has published the current one, so
//     a whole hand-back period of the stage (several microseconds) hides the memory latency, and as many tiles as
//     there are scatter warps are in flight per CTA.  No copy ring, no producer warps, no per-chunk barriers.
//   * A stage is cleared with 32 16-byte stores per lane: clearing only the cells the previous tile wrote (their
//     locations kept in registers) takes more, and slower, store instructions and measured slower.  Tiles with more vectors than the register budget (CAP per lane) fetch and scatter
//     the excess in a plain loop.
#pragma once
#include "spmm_kernel_sm100.cuh"

namespace flashllm {

__device__ __forceinline__ uint4 ldg_stream16(const uint4* ptr)
{
    uint4 v;
#ifndef FLASHLLM_LDG_FLAVOUR
#define FLASHLLM_LDG_FLAVOUR "ld.global.nc.L1::no_allocate.v4.u32"
#endif
    asm volatile(FLASHLLM_LDG_FLAVOUR " {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(ptr));
    return v;
}

// Straight-line forms for the scatter warps' per-tile path.  That path is bound by the number of instructions and
// branches a warp has to get through per tile, so a row of 32 vectors is loaded / scattered by predicated instructions
// behind ONE comparison (`rem` = vectors of the tile from this lane's first one on, against the row's constant offset)
// instead of being guarded by branches, and row addresses are one base register plus a constant.
template<int VEC_OFFSET>
__device__ __forceinline__ void ldg_row_if(uint4& v, const uint4* lane_base, int rem)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.gt.s32 p, %5, %6;\n"
        "@p " FLASHLLM_LDG_FLAVOUR " {%0, %1, %2, %3}, [%4 + %7];\n"
        "}\n"
        : "+r"(v.x), "+r"(v.y), "+r"(v.z), "+r"(v.w)
        : "l"(lane_base), "r"(rem), "n"(VEC_OFFSET), "n"(VEC_OFFSET * 16));
}

template<int VEC_OFFSET>
__device__ __forceinline__ void scatter_row_if(uint32_t stage, const uint4& w, int rem)
{
    const uint32_t a0 = stage + ((w.x >> 15) & 0x3FFEu), a1 = stage + ((w.y >> 15) & 0x3FFEu);
    const uint32_t a2 = stage + ((w.z >> 15) & 0x3FFEu), a3 = stage + ((w.w >> 15) & 0x3FFEu);
#if (FLASHLLM_ABLATE & 32)  // timing only: whole-word stores in place of the 16-bit ones (neighbours get clobbered)
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.gt.s32 p, %8, %9;\n"
        "@p st.shared.u32 [%0], %4;\n"
        "@p st.shared.u32 [%1], %5;\n"
        "@p st.shared.u32 [%2], %6;\n"
        "@p st.shared.u32 [%3], %7;\n"
        "}\n" ::"r"(a0 & ~3u),
        "r"(a1 & ~3u), "r"(a2 & ~3u), "r"(a3 & ~3u), "r"(w.x << 16), "r"(w.y << 16), "r"(w.z << 16), "r"(w.w << 16), "r"(rem),
        "n"(VEC_OFFSET)
        : "memory");
    return;
#endif
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.gt.s32 p, %8, %9;\n"
        "@p st.shared.u16 [%0], %4;\n"
        "@p st.shared.u16 [%1], %5;\n"
        "@p st.shared.u16 [%2], %6;\n"
        "@p st.shared.u16 [%3], %7;\n"
        "}\n" ::"r"(a0),
        "r"(a1), "r"(a2), "r"(a3), "h"(static_cast<unsigned short>(w.x & 0xFFFFu)),
        "h"(static_cast<unsigned short>(w.y & 0xFFFFu)), "h"(static_cast<unsigned short>(w.z & 0xFFFFu)),
        "h"(static_cast<unsigned short>(w.w & 0xFFFFu)), "r"(rem), "n"(VEC_OFFSET)
        : "memory");
}

// Rows [FIRST, LAST) of a warp's share of a tile: the warp's row q is the tile's row q * WPT + its index among the
// WPT warps that share the tile (already folded into lane_base and rem).
template<int FIRST, int LAST, int WPT, int CAP>
__device__ __forceinline__ void load_rows(uint4 (&buf)[CAP], const uint4* lane_base, int rem)
{
    if constexpr (FIRST < LAST) {
        ldg_row_if<FIRST * WPT * 32>(buf[FIRST], lane_base, rem);
        load_rows<FIRST + 1, LAST, WPT, CAP>(buf, lane_base, rem);
    }
}

template<int FIRST, int LAST, int WPT, int CAP>
__device__ __forceinline__ void scatter_rows(uint32_t stage, const uint4 (&buf)[CAP], int rem)
{
    if constexpr (FIRST < LAST) {
        scatter_row_if<FIRST * WPT * 32>(stage, buf[FIRST], rem);
        scatter_rows<FIRST + 1, LAST, WPT, CAP>(stage, buf, rem);
    }
}

// A warp's batch of up to CAP rows: the lower half always, the upper half only when the tile reaches it (one branch),
// so that sparse tiles do not pay for rows they do not have.
template<int WPT, int CAP>
__device__ __forceinline__ void load_batch(uint4 (&buf)[CAP], const uint4* lane_base, int rem_uniform, int rem)
{
    load_rows<0, CAP / 2, WPT, CAP>(buf, lane_base, rem);
    if (rem_uniform > (CAP / 2) * WPT * 32)
        load_rows<CAP / 2, CAP, WPT, CAP>(buf, lane_base, rem);
}

template<int WPT, int CAP>
__device__ __forceinline__ void scatter_batch(uint32_t stage, const uint4 (&buf)[CAP], int rem_uniform, int rem)
{
    scatter_rows<0, CAP / 2, WPT, CAP>(stage, buf, rem);
    if (rem_uniform > (CAP / 2) * WPT * 32)
        scatter_rows<CAP / 2, CAP, WPT, CAP>(stage, buf, rem);
}

// How many of its own tiles ahead a scatter warp asks the memory system to bring into L2 (its register loads run one
// tile ahead).
#ifndef FLASHLLM_PREFETCH_AHEAD
#define FLASHLLM_PREFETCH_AHEAD 2
#endif
constexpr int kPrefetchAhead = FLASHLLM_PREFETCH_AHEAD;

// Warps of the register-streaming kernel: one B loader, kDirectIssuers MMA issuers, then the scatter warps.
constexpr int kDirectIssuers = 2;

// CAP: vectors per lane kept in registers.  WARPS: stages = tiles in flight per CTA.  WPT: warps that share one tile
// (row q of warp h is the tile's row q * WPT + h), so a tile of up to 32 * CAP * WPT vectors is handled without the
// overflow loop and a warp's instruction stream per tile is 1 / WPT as long.  MIN_BLOCKS: CTAs per SM the register
// budget is sized for.
//
// One thread cannot issue tcgen05.mma as fast as the tensor core retires them (measured: 4 MMAs and the commit that
// hands a stage back cost an issuing thread ~400 cycles, the tensor core ~180), so tiles alternate between
// kDirectIssuers issuing threads, each with an accumulator of its own in tensor memory; the epilogue adds them.
template<int N_TILE, int CAP, int WARPS, int MIN_BLOCKS, int WPT = 1>
__global__ void __launch_bounds__((1 + kDirectIssuers + WARPS * WPT) * 32, MIN_BLOCKS)
    spmm_tcgen05_direct_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    static_assert(WARPS >= 4 && WARPS <= 12, "four warps cover the TMEM lane quarters in the epilogue");
    static_assert(WPT == 1 || WPT == 2, "a tile is decompressed by one warp or by a pair");
    static_assert(CAP % 2 == 0 && 32 % WPT == 0, "batches are issued in two halves; the clear is split evenly");
    constexpr uint32_t kBSlab    = N_TILE * kTileK * 2;  // one K tile of B in shared memory
    constexpr int      MI        = kDirectIssuers;
    static_assert(WARPS % MI == 0, "every issuer serves the same stages on every lap");
    constexpr uint32_t kTmemCols = MI * N_TILE < 32 ? 32 : MI * N_TILE;  // a power of two for MI = 2
    constexpr int      NSW       = WARPS * WPT;  // scatter warps
    constexpr int      a_stages  = WARPS;

#ifdef FLASHLLM_TRACE
    __shared__ unsigned int s_trace[kTraceKinds * kTraceDepth];
    for (int i = threadIdx.x; i < kTraceKinds * kTraceDepth; i += blockDim.x)
        s_trace[i] = 0;
#endif
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base     = (raw_addr + 1023u) & ~1023u;  // swizzled operands need 1024-byte alignment
    uint8_t* const smem     = smem_raw + (base - raw_addr);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    if (threadIdx.x == 0)
        FL_CTA_TIME(0);

    const SpmmPlan& plan     = p.plan;
    const int       b_stages = plan.b_stages;
    const int       KB       = plan.b_batch;
    const int       S        = plan.cluster_k;
    const int       G        = plan.workspace_k;
    constexpr int   b_warp   = 0;  // warp that loads B
    constexpr int   mma_warp = 1;       // first of the MI warps that issue MMAs; it owns the TMEM allocation
    constexpr int   first_sw = 1 + MI;  // first scatter warp
    constexpr int   NTS      = NSW * 32;

    // ---- shared memory carve-up
    const uint32_t a_base   = base;
    const uint32_t b_base   = a_base + a_stages * kDenseTileBytes;
    const uint32_t bar_base = b_base + b_stages * KB * kBSlab;
    const uint32_t a_full   = bar_base;
    const uint32_t a_empty  = a_full + 8u * a_stages;
    const uint32_t b_full   = a_empty + 8u * a_stages;
    const uint32_t b_empty  = b_full + 8u * b_stages;
    const uint32_t acc_full = b_empty + 8u * b_stages;
    const uint32_t misc_off = (acc_full + 8u) - base;
    volatile uint32_t* const tmem_slot  = reinterpret_cast<volatile uint32_t*>(smem + misc_off);
    volatile uint32_t* const abort_flag = reinterpret_cast<volatile uint32_t*>(smem + misc_off + 4);
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

    // ---- scatter warps: the first tile's words are requested before anything else, so that the set-up below
    // (barrier initialisation, tensor-memory allocation, offset staging and checking: ~1.5 us) hides behind their
    // latency instead of preceding it.  The two offsets are read straight from global memory and checked on the spot.
    const int sw        = warp - first_sw;
    const int st        = sw % WARPS;       // the stage, and the tile stream st, st + WARPS, ... this warp works on
    const int h         = sw / WARPS;       // its index among the WPT warps that share those tiles
    const int first_vec = h * 32 + lane;    // this lane's vector in row 0 of the warp's share
    uint4     nxt[CAP];                     // words of the tile about to be scattered (loads in flight)
    int          n_in = 0;                  // vectors of the whole tile whose share is in nxt
    const uint4* src  = p.compressed;
    bool         bad  = false;
    if (warp >= first_sw) {
#pragma unroll
        for (int q = 0; q < CAP; ++q)
            nxt[q] = make_uint4(0u, 0u, 0u, 0u);
        if (st < L) {
            const int vb = offs_global[st], ve = offs_global[st + 1];
            bad          = (ve < vb) || (ve - vb > kMaxTileVectors) || (vb < 0);
            n_in         = bad ? 0 : ve - vb;
            src          = p.compressed + (bad ? 0 : vb);
            load_batch<WPT, CAP>(nxt, src + first_vec, n_in, n_in - first_vec);
        }
    }

    // ---- set-up
    if (threadIdx.x == 0) {
        for (int i = 0; i < a_stages; ++i) {
            ptx::mbar_init(a_full + 8u * i, WPT);  // every warp that shares the tile publishes its part
            ptx::mbar_init(a_empty + 8u * i, 1);
        }
        for (int i = 0; i < b_stages; ++i) {
            ptx::mbar_init(b_full + 8u * i, 1);
            ptx::mbar_init(b_empty + 8u * i, MI);  // every issuer hands a batch back
        }
        ptx::mbar_init(acc_full, MI);
        abort_flag[0]             = 0u;  // a launch never inherits a give-up from an earlier one: the status word only reports
        abort_flag[kDepsResolved] = 0u;
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
    // A following kernel of this library may start its set-up and weight streaming while this grid drains; it waits
    // (in its B loader) before it touches anything this grid or its predecessors produce.
    if (threadIdx.x == 0)
        ptx::grid_launch_dependents();
    if (threadIdx.x == 0)
        FL_CTA_TIME(1);

    if (warp == b_warp) {
        // ================================================================ B loader: KB K tiles per TMA instruction
        if (lane == 0 && L > 0 && go) {
            load_b_batches(&tmap_b, (L + KB - 1) / KB, KB, b_stages, kBSlab, b_base, b_full, b_empty, n_idx * N_TILE, k_begin,
                           abort_flag, p.status);
        }
    }
    else if (warp < first_sw) {
        // ================================================================ MMA issuers: issuer m takes tiles m, m + MI, ...
        // The B batches hold a multiple of MI tiles, so every issuer has work in every full batch and hands it back
        // itself; the last, partial batch is never waited for.
        if (lane == 0 && go) {
            const int m = warp - mma_warp;
            if (m < L) {
                const uint32_t idesc   = ptx::umma_idesc_f16_f32(kTileM, N_TILE);
                const uint64_t a_desc0 = ptx::umma_desc_kmajor_sw128(a_base);
                const uint64_t b_desc0 = ptx::umma_desc_kmajor_sw128(b_base);
                const uint32_t acc     = tmem_acc + static_cast<uint32_t>(m * N_TILE);
                int            s = m, bs = 0, kb = m;
                uint32_t       a_par = 0, b_par = 0;
                bool           ready = false, first_in_batch = true;
                for (int j = m; j < L; j += MI) {
                    if (m == 0)
                        FL_TRACE(7, j);
                    if (!ready) {
                        if (!wait_bounded(a_full + 8u * s, a_par, abort_flag, p.status))
                            break;
                        if (first_in_batch && !wait_bounded(b_full + 8u * bs, b_par, abort_flag, p.status))
                            break;
                    }
                    if (m == 0)
                        FL_TRACE(9, j);
                    int      s_n = s + MI, kb_n = kb + MI, bs_n = bs;
                    uint32_t a_par_n = a_par, b_par_n = b_par;
                    if (s_n >= a_stages) {
                        s_n -= a_stages;
                        a_par_n ^= 1u;
                    }
                    const bool batch_done = kb_n >= KB;
                    if (batch_done) {
                        kb_n -= KB;
                        if (++bs_n == b_stages) {
                            bs_n = 0;
                            b_par_n ^= 1u;
                        }
                    }
                    const bool has_next = j + MI < L;
                    ptx::tc_fence_after_sync();
#if (FLASHLLM_ABLATE & 4)
                    ptx::umma_commit(a_empty + 8u * s);  // timing only: hand-backs without any MMA
                    if (batch_done || !has_next)
                        ptx::umma_commit(b_empty + 8u * bs);
                    ready = false;
                    if (false)
#endif
                    ready = ptx::umma_tile_commit_probe(
                        acc, a_desc0 + static_cast<uint32_t>(s * (kDenseTileBytes >> 4)),
                        b_desc0 + static_cast<uint32_t>((bs * KB + kb) * (kBSlab >> 4)), idesc, j != m ? 1u : 0u, a_empty + 8u * s,
                        b_empty + 8u * bs, (batch_done || !has_next) ? 1u : 0u, a_full + 8u * s_n, a_par_n, b_full + 8u * bs_n,
                        b_par_n, has_next ? 1u : 0u, (has_next && batch_done) ? 1u : 0u);
                    if (m == 0)
                        FL_TRACE(10, j);
                    first_in_batch = batch_done;
                    s     = s_n;
                    kb    = kb_n;
                    bs    = bs_n;
                    a_par = a_par_n;
                    b_par = b_par_n;
                }
            }
            ptx::umma_commit(acc_full);
        }
    }
    else {
        // ================================================================ scatter warps: WPT warps per stage
        if (L > 0 && go) {
            const uint32_t stage     = a_base + st * kDenseTileBytes;
            const uint32_t full_bar  = a_full + 8u * st;
            const uint32_t empty_bar = a_empty + 8u * st;
            // the tile after the first one is pulled from DRAM into L2 (its register loads come one tile from now)
            if (st < L && lane == 0 && h == 0) {
                for (int a = 1; a < kPrefetchAhead; ++a) {
                    const int t = st + a * WARPS;
                    if (t < L && offs[t + 1] > offs[t])
                        ptx::prefetch_l2_bulk(p.compressed + offs[t], static_cast<uint32_t>(offs[t + 1] - offs[t]) * 16u);
                }
            }
            uint32_t use = 0;
            for (int j = st; j < L; j += WARPS, ++use) {
                if (bad)
                    atomicOr(p.status, kStatusBadTileOffsets);
                if (lane == 0)
                    FL_TRACE(0, j);
                bool ok = !bad;
                if (ok && use > 0)
                    ok = wait_bounded_warp(empty_bar, (use & 1u) ^ 1u, abort_flag, p.status);
                if (!ok) {  // uniform across the warps that share the tile: they watch the same barrier and flag
                    if (bad)
                        *abort_flag = 1u;
                    break;
                }
                if (lane == 0)
                    FL_TRACE(3, j);
                // Offsets of this warp's following tile.  Two places are wrong for these two shared-memory loads: right
                // behind the previous tile's global loads (they queue behind them in the load/store unit: ~700 cycles at
                // the loop's top) and behind the proxy fence below (they wait for it, and the loads that need them wait
                // for them: the refill then takes ~7000 cycles instead of ~650).  Here the unit is idle.
                const bool has_next = j + WARPS < L;
                int        vb2 = 0, ve2 = 0;
                if (has_next) {
                    vb2 = offs[j + WARPS];
                    ve2 = offs[j + WARPS + 1];
                }
                // ---- clear the stage (each sharing warp its part), then scatter the new tile
                if (!(FLASHLLM_ABLATE & 1)) {
#pragma unroll
                    for (int q = 0; q < 32 / WPT; ++q)
                        sts_zero16(stage + static_cast<uint32_t>((q * WPT + h) * 32 + lane) * 16u);
                }
                // another lane's (or the partner warp's) zero must not land on top of a new value
                if (WPT == 1)
                    __syncwarp();
                else
                    ptx::named_barrier_sync(1u + static_cast<uint32_t>(st), 32u * WPT);
                if (lane == 0)
                    FL_TRACE(2, j);
                {
                    const int rem = n_in - first_vec;
#if (FLASHLLM_ABLATE & 2)
#pragma unroll
                    for (int q = 0; q < CAP; ++q)
                        if ((nxt[q].x ^ nxt[q].y ^ nxt[q].z ^ nxt[q].w) == 0x9E3779B9u)  // keeps the loads alive
                            scatter_word(stage, nxt[q].x);
#else
                    scatter_batch<WPT, CAP>(stage, nxt, n_in, rem);
#endif
                    // tiles denser than the register budget: the rest in further batches, fetched only now
                    for (int v0 = CAP * WPT * 32; v0 < n_in; v0 += CAP * WPT * 32) {
                        load_batch<WPT, CAP>(nxt, src + v0 + first_vec, n_in - v0, rem - v0);
                        scatter_batch<WPT, CAP>(stage, nxt, n_in - v0, rem - v0);
                    }
                }
                if (lane == 0)
                    FL_TRACE(5, j);
#if !(FLASHLLM_ABLATE & 16)  // timing only: without the proxy fence the tensor core may read stale words
                ptx::fence_proxy_async_smem();
#endif
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(full_bar);
                if (lane == 0)
                    FL_TRACE(6, j);
                // ---- start fetching the following tile
                if (has_next) {
                    bad  = (ve2 < vb2) || (ve2 - vb2 > kMaxTileVectors) || (vb2 < 0);
                    n_in = bad ? 0 : ve2 - vb2;
                    src  = p.compressed + (bad ? 0 : vb2);
                    if (!(FLASHLLM_ABLATE & 8))
                        load_batch<WPT, CAP>(nxt, src + first_vec, n_in, n_in - first_vec);
                    // ... and pull the one after it from DRAM into L2, so that its register loads, issued one tile
                    // from now, only have the L2 latency left to hide
                    if (lane == 0 && h == 0 && j + kPrefetchAhead * WARPS < L) {
                        const int pb = offs[j + kPrefetchAhead * WARPS], pe = offs[j + kPrefetchAhead * WARPS + 1];
                        if (pe > pb)
                            ptx::prefetch_l2_bulk(p.compressed + pb, static_cast<uint32_t>(pe - pb) * 16u);
                    }
                }
                if (lane == 0)
                    FL_TRACE(13, j);
            }
        }

        // ================================================================ epilogue (same warps)
        bool acc_ok = go;
        if (L > 0 && go)
            acc_ok = wait_bounded_warp(acc_full, 0u, abort_flag, p.status);
        acc_ok = __all_sync(0xFFFFFFFFu, acc_ok && (*abort_flag == 0u));
        ptx::tc_fence_after_sync();
        if (sw == 0 && lane == 0)
            FL_CTA_TIME(2);

        accumulators_to_output<N_TILE>(p, tmem_acc, L < MI ? L : MI, N_TILE, warp & 3, lane, sw, NSW >= 8 ? 2 : 1, S, G, g,
                                       n_idx, tile_row, acc_ok, reinterpret_cast<float*>(smem));
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
    if (threadIdx.x == 0)
        FL_CTA_TIME(3);
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

}  // namespace flashllm
