// Load-as-Sparse / Compute-as-Dense SpMM for sm_100a, register-streaming form with a janitor warp.
//
// Same work split as the register-streaming form (one CTA = one 128-row tile row x one N tile x a K range; B loader,
// two MMA issuers with an accumulator each, scatter warps that fetch a whole tile into registers with 16-byte global
// loads and also run the epilogue), with the per-stage chain "wait for the stage -> clear -> scatter -> publish ->
// refill" taken apart:
//
//   * Stages are cleared by a warp of their own, the janitor: it waits for the commit that hands a stage back, fills
//     it with zeros (32 16-byte stores per lane) and signals an mbarrier the next scatter warp waits on.  The clear is
//     off the scatter warps' chain and overlaps their work on other stages, and a scatter warp's loads for its next
//     tile are in flight while the multiply and the clear of its previous one run.  (Clearing with the TMA unit -- a
//     tensor copy whose box lies wholly outside its tensor writes the fill value without reading global memory -- was
//     measured: one 16 KB fill every ~900 cycles per SM however many are in flight, three times too slow.  The
//     reference clears with zero-size cp.async, csrc/SpMM_Kernel.cuh:114-136.)
//   * Stages are decoupled from warps (tile j lives in stage j mod a_stages, a_stages >= WARPS): with spare stages a
//     warp that has published a tile goes on with its next one instead of waiting for its own stage to come back.
//   * Six scatter warps per CTA, two CTAs per SM, is the default shape: a tile's loads are issued as one batch and
//     consumed as one batch (a window refilled row by row was measured at a third of the speed: the hardware tracks
//     outstanding loads with a handful of counters per warp, and waiting for an old load then also waits for the young
//     ones that share its counter), so what keeps the memory system busy is the number of warps with a batch in flight.
#pragma once
#include "spmm_kernel_direct_sm100.cuh"

namespace flashllm {

// Warps of the continuous-stream kernel: B loader, janitor, kDirectIssuers MMA issuers, then the scatter warps.
template<int N_TILE, int CAP, int WARPS, int MIN_BLOCKS>
__global__ void __launch_bounds__((2 + kDirectIssuers + WARPS) * 32, MIN_BLOCKS)
    spmm_tcgen05_janitor_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    static_assert(WARPS >= 4 && WARPS <= 12, "four warps cover the TMEM lane quarters in the epilogue");
    constexpr uint32_t kBSlab    = N_TILE * kTileK * 2;  // one K tile of B in shared memory
    constexpr int      MI        = kDirectIssuers;
    constexpr uint32_t kTmemCols = MI * N_TILE < 32 ? 32 : MI * N_TILE;  // a power of two for MI = 2
    constexpr int      NSW       = WARPS;

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

    const SpmmPlan& plan     = p.plan;
    const int       a_stages = plan.a_stages;
    const int       b_stages = plan.b_stages;
    const int       KB       = plan.b_batch;
    const int       S        = plan.cluster_k;
    const int       G        = plan.workspace_k;
    constexpr int   b_warp   = 0;  // loads B
    constexpr int   z_warp   = 1;  // janitor: clears stages that have been handed back
    constexpr int   mma_warp = 2;  // first of the MI warps that issue MMAs; it owns the TMEM allocation
    constexpr int   first_sw = 2 + MI;
    constexpr int   NTS      = NSW * 32;

    // ---- shared memory carve-up
    const uint32_t a_base   = base;
    const uint32_t b_base   = a_base + a_stages * kDenseTileBytes;
    const uint32_t bar_base = b_base + b_stages * KB * kBSlab;
    const uint32_t a_full   = bar_base;                  // scatter warp -> MMA issuer: tile decompressed
    const uint32_t a_empty  = a_full + 8u * a_stages;    // MMA commit -> janitor: stage read, may be cleared
    const uint32_t a_zero   = a_empty + 8u * a_stages;   // janitor -> scatter warp: stage holds zeros
    const uint32_t b_full   = a_zero + 8u * a_stages;
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

    // ---- set-up
    if (threadIdx.x == 0) {
        for (int i = 0; i < a_stages; ++i) {
#ifdef FLASHLLM_LANE_ARRIVE
            ptx::mbar_init(a_full + 8u * i, 32);  // every lane of the scatter warp arrives for itself
#else
            ptx::mbar_init(a_full + 8u * i, 1);
#endif
            ptx::mbar_init(a_empty + 8u * i, 1);
            ptx::mbar_init(a_zero + 8u * i, 1);
        }
        for (int i = 0; i < b_stages; ++i) {
            ptx::mbar_init(b_full + 8u * i, 1);
            ptx::mbar_init(b_empty + 8u * i, MI);  // every issuer hands a batch back
        }
        ptx::mbar_init(acc_full, MI);
        abort_flag[0]             = 0u;
        abort_flag[kDepsResolved] = 0u;  // set once the B loader has passed the grid dependency
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
    const bool go = !bad_slice;  // false: every role skips its work and nothing is stored
    if (bad_slice && threadIdx.x == 0) {
        atomicOr(p.status, kStatusBadTileOffsets);
        *abort_flag = 1u;
    }
    const uint32_t tmem_acc = *tmem_slot;
    // A following kernel of this library may start its set-up and weight streaming while this grid drains; it waits
    // (in its B loader) before it touches anything this grid or its predecessors produce.
    if (threadIdx.x == 0)
        ptx::grid_launch_dependents();

    if (warp == b_warp) {
        // ================================================================ B loader: KB K tiles per TMA instruction
        if (lane == 0 && L > 0 && go) {
            load_b_batches(&tmap_b, (L + KB - 1) / KB, KB, b_stages, kBSlab, b_base, b_full, b_empty, n_idx * N_TILE, k_begin,
                           abort_flag, p.status);
        }
    }
    else if (warp == z_warp) {
        // ================================================================ janitor: clears stages that were handed back
#ifdef FLASHLLM_SELF_CLEAR
        if (false) {
#else
        if (L > 0 && go) {
#endif
            const int first = L < a_stages ? L : a_stages;
            for (int s = 0; s < first; ++s) {  // every stage starts out cleared
                zero_fill_stage(a_base + s * kDenseTileBytes, lane);
#ifdef FLASHLLM_JANITOR_FENCE
                ptx::fence_proxy_async_smem();
#endif
                __syncwarp();  // every lane's stores precede lane 0's release
                if (lane == 0)
                    ptx::mbar_arrive(a_zero + 8u * s);
            }
            int      s   = 0;
            uint32_t par = 0;
            for (int j = 0; j + a_stages < L; ++j) {  // tile j's stage is reused by tile j + a_stages
                if (lane == 0)
                    FL_TRACE(14, j);
                if (!wait_bounded_warp(a_empty + 8u * s, par, abort_flag, p.status))
                    break;
                if (lane == 0)
                    FL_TRACE(15, j);
                zero_fill_stage(a_base + s * kDenseTileBytes, lane);
#ifdef FLASHLLM_JANITOR_FENCE
                ptx::fence_proxy_async_smem();
#endif
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(a_zero + 8u * s);
                if (lane == 0)
                    FL_TRACE(16, j);
                if (++s == a_stages) {
                    s = 0;
                    par ^= 1u;
                }
            }
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
                int            s = m % a_stages, bs = 0, kb = m;
                uint32_t       a_par = static_cast<uint32_t>(m / a_stages) & 1u, b_par = 0;
                bool           ready = false, first_in_batch = true;
                for (int j = m; j < L; j += MI) {
                    FL_TRACE(7, j);
                    if (!ready) {
                        if (!wait_bounded(a_full + 8u * s, a_par, abort_flag, p.status))
                            break;
                        if (first_in_batch && !wait_bounded(b_full + 8u * bs, b_par, abort_flag, p.status))
                            break;
                    }
                    FL_TRACE(9, j);
                    int      s_n = s + MI, kb_n = kb + MI, bs_n = bs;
                    uint32_t a_par_n = a_par, b_par_n = b_par;
                    while (s_n >= a_stages) {
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
#ifdef FLASHLLM_CONSUMER_FENCE
                    // Variant: the proxy fence on the consuming side.  The scatter warp's generic-proxy stores were
                    // published with a release on a_full, which this thread has observed; the fence then orders them
                    // before the tensor core's async-proxy reads of the stage.
                    ptx::fence_proxy_async_smem();
#endif
                    ptx::tc_fence_after_sync();
                    ready = ptx::umma_tile_commit_probe(
                        acc, a_desc0 + static_cast<uint32_t>(s * (kDenseTileBytes >> 4)),
                        b_desc0 + static_cast<uint32_t>((bs * KB + kb) * (kBSlab >> 4)), idesc, j != m ? 1u : 0u, a_empty + 8u * s,
                        b_empty + 8u * bs, (batch_done || !has_next) ? 1u : 0u, a_full + 8u * s_n, a_par_n, b_full + 8u * bs_n,
                        b_par_n, has_next ? 1u : 0u, (has_next && batch_done) ? 1u : 0u);
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
        // ================================================================ scatter warps
        const int sw = warp - first_sw;
        if (sw < L && go) {
            uint4 nxt[CAP];  // words of the tile about to be scattered (loads in flight)
#pragma unroll
            for (int q = 0; q < CAP; ++q)
                nxt[q] = make_uint4(0u, 0u, 0u, 0u);
            int          n_in = 0;  // vectors of the tile in nxt
            const uint4* src  = p.compressed;
            // Requests the first CAP rows (32 vectors each) of a tile as one batch; rows past the tile's end are
            // skipped by real branches, not issued predicated off.
            auto fetch = [&](int vb, int ve, int t) {
                int n = ve - vb;
                n     = n < 0 ? 0 : (n > kMaxTileVectors ? kMaxTileVectors : n);  // the slice was validated at set-up
                n_in  = n;
                src   = p.compressed + vb;
#pragma unroll
                for (int q = 0; q < CAP; ++q) {
                    if (q * 32 >= n)
                        break;
                    if (q * 32 + lane < n)
                        nxt[q] = ldg_stream16(src + q * 32 + lane);
                }
                // ... and a later tile of this warp is pulled from DRAM into L2, so that its register loads, issued
                // a tile or two from now, only have the L2 latency left to hide
                if (lane == 0) {
                    const int a = t + kPrefetchAhead * NSW;
                    if (a < L && offs[a + 1] > offs[a])
                        ptx::prefetch_l2_bulk(p.compressed + offs[a], static_cast<uint32_t>(offs[a + 1] - offs[a]) * 16u);
                }
            };
            fetch(offs[sw], offs[sw + 1], sw);
            if (lane == 0 && sw + NSW < L && offs[sw + NSW + 1] > offs[sw + NSW])
                ptx::prefetch_l2_bulk(p.compressed + offs[sw + NSW],
                                      static_cast<uint32_t>(offs[sw + NSW + 1] - offs[sw + NSW]) * 16u);

            int      s_idx = sw % a_stages;                                // stage of tile j ...
            uint32_t s_par = static_cast<uint32_t>(sw / a_stages) & 1u;    // ... and which use of it
            for (int j = sw; j < L; j += NSW) {
                // Offsets of this warp's following tile, read before the proxy fence below: a shared-memory load
                // issued behind that fence waits for it.
                const bool has_next = j + NSW < L;
                int        vb2 = 0, ve2 = 0;
                if (has_next) {
                    vb2 = offs[j + NSW];
                    ve2 = offs[j + NSW + 1];
                }
                if (lane == 0)
                    FL_TRACE(0, j);
                const uint32_t stage = a_base + static_cast<uint32_t>(s_idx) * kDenseTileBytes;
#ifdef FLASHLLM_SELF_CLEAR
                if (j >= a_stages && !wait_bounded_warp(a_empty + 8u * s_idx, s_par ^ 1u, abort_flag, p.status))
                    break;
                zero_fill_stage(stage, lane);
                __syncwarp();
#else
                if (!wait_bounded_warp(a_zero + 8u * s_idx, s_par, abort_flag, p.status))
                    break;
#endif
                if (lane == 0)
                    FL_TRACE(3, j);
                const int      n_reg = n_in < CAP * 32 ? n_in : CAP * 32;
#pragma unroll
                for (int q = 0; q < CAP; ++q) {
                    if (q * 32 >= n_reg)
                        break;
                    if (q * 32 + lane < n_reg)
                        scatter_vector(stage, nxt[q]);
                }
                // tiles denser than the register budget: the rest in further batches, fetched only now
                for (int v0 = n_reg; v0 < n_in; v0 += CAP * 32) {
#pragma unroll
                    for (int q = 0; q < CAP; ++q) {
                        if (v0 + q * 32 >= n_in)
                            break;
                        if (v0 + q * 32 + lane < n_in)
                            nxt[q] = ldg_stream16(src + v0 + q * 32 + lane);
                    }
#pragma unroll
                    for (int q = 0; q < CAP; ++q) {
                        if (v0 + q * 32 >= n_in)
                            break;
                        if (v0 + q * 32 + lane < n_in)
                            scatter_vector(stage, nxt[q]);
                    }
                }
                if (lane == 0)
                    FL_TRACE(5, j);
#ifdef FLASHLLM_FETCH_FIRST
                if (has_next)
                    fetch(vb2, ve2, j + NSW);
#endif
#ifndef FLASHLLM_CONSUMER_FENCE
                ptx::fence_proxy_async_smem();  // generic-proxy stores (the janitor's zeros, observed through a_zero,
                                                // and this warp's words) -> the tensor core's async-proxy reads
#endif
                if (lane == 0)
                    FL_TRACE(17, j);
#ifdef FLASHLLM_LANE_ARRIVE
                ptx::mbar_arrive(a_full + 8u * s_idx);
#else
                __syncwarp();  // every lane's stores precede lane 0's release
                if (lane == 0)
                    FL_TRACE(18, j);
                if (lane == 0)
                    ptx::mbar_arrive(a_full + 8u * s_idx);
#endif
                if (lane == 0)
                    FL_TRACE(6, j);
#ifndef FLASHLLM_FETCH_FIRST
                if (has_next)
                    fetch(vb2, ve2, j + NSW);
#endif
                s_idx += NSW;
                while (s_idx >= a_stages) {
                    s_idx -= a_stages;
                    s_par ^= 1u;
                }
            }
        }

        // ================================================================ epilogue (same warps)
        bool acc_ok = go;
        if (L > 0 && go)
            acc_ok = wait_bounded_warp(acc_full, 0u, abort_flag, p.status);
        acc_ok = __all_sync(0xFFFFFFFFu, acc_ok && (*abort_flag == 0u));
        ptx::tc_fence_after_sync();

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
    push_raise_flags(p, *abort_flag == 0u);
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
