// Load-as-Sparse / Compute-as-Dense SpMM for sm_100a, continuous-stream form.
//
// Same work split as the register-streaming form (one CTA = one 128-row tile row x one N tile x a K range; B loader,
// two MMA issuers with an accumulator each, scatter warps that also run the epilogue), with three changes that take
// the per-stage chain "wait for the stage -> clear -> scatter -> publish -> refill" apart:
//
//   * A scatter warp treats the tiles it owns (w, w + WARPS, ...) as ONE stream of 32-vector rows and keeps CAP rows of
//     it in registers as a circular window: as soon as a row has been scattered, the register it sat in is refilled
//     with the row CAP places further down the stream, whichever tile that belongs to.  Global loads are therefore in
//     flight all the time (CAP x 512 bytes per warp), not only between a publish and the next scatter, and tiles of any
//     density go through the same path (the reference keeps a whole tile in registers, csrc/SpMM_Kernel.cuh:17-62,
//     which caps a tile at 4096 non-zeros).
//   * Stages are cleared by a warp of their own, the janitor: it waits for the commit that hands a stage back, fills
//     it with zeros (32 16-byte stores per lane) and signals an mbarrier the next scatter warp waits on.  The clear is
//     thereby off the scatter warps' chain and overlaps their work on other stages.  (Clearing with the TMA unit -- a
//     tensor copy whose box lies wholly outside its tensor writes the fill value without reading global memory -- was
//     measured: one 16 KB fill every ~900 cycles per SM however many are in flight, three times too slow.  The
//     reference clears with zero-size cp.async, csrc/SpMM_Kernel.cuh:114-136.)
//   * Stages are decoupled from warps (tile j lives in stage j mod a_stages, a_stages >= WARPS): a warp that has
//     published a tile goes on with its next one in another stage instead of waiting for its own stage to come back.
#pragma once
#include "spmm_kernel_direct_sm100.cuh"

namespace flashllm {

// Warps of the continuous-stream kernel: B loader, janitor, kDirectIssuers MMA issuers, then the scatter warps.
template<int N_TILE, int CAP, int WARPS, int MIN_BLOCKS>
__global__ void __launch_bounds__((2 + kDirectIssuers + WARPS) * 32, MIN_BLOCKS)
    spmm_tcgen05_stream_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    static_assert(WARPS >= 4 && WARPS <= 12, "four warps cover the TMEM lane quarters in the epilogue");
    constexpr uint32_t kBSlab    = N_TILE * kTileK * 2;  // one K tile of B in shared memory
    constexpr int      MI        = kDirectIssuers;
    constexpr uint32_t kTmemCols = MI * N_TILE < 32 ? 32 : MI * N_TILE;  // a power of two for MI = 2
    constexpr int      NSW       = WARPS;

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
            ptx::mbar_init(a_full + 8u * i, 1);
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
        if (L > 0 && go) {
            const int first = L < a_stages ? L : a_stages;
            for (int s = 0; s < first; ++s) {  // every stage starts out cleared
                zero_fill_stage(a_base + s * kDenseTileBytes, lane);
                __syncwarp();  // every lane's stores precede lane 0's release
                if (lane == 0)
                    ptx::mbar_arrive(a_zero + 8u * s);
            }
            int      s   = 0;
            uint32_t par = 0;
            for (int j = 0; j + a_stages < L; ++j) {  // tile j's stage is reused by tile j + a_stages
                if (!wait_bounded_warp(a_empty + 8u * s, par, abort_flag, p.status))
                    break;
                zero_fill_stage(a_base + s * kDenseTileBytes, lane);
                __syncwarp();
                if (lane == 0)
                    ptx::mbar_arrive(a_zero + 8u * s);
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
                    if (!ready) {
                        if (!wait_bounded(a_full + 8u * s, a_par, abort_flag, p.status))
                            break;
                        if (first_in_batch && !wait_bounded(b_full + 8u * bs, b_par, abort_flag, p.status))
                            break;
                    }
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
            uint4 win[CAP];  // the window: rows i, i+1, ... of this warp's stream, row r in win[r mod CAP]
#pragma unroll
            for (int q = 0; q < CAP; ++q)
                win[q] = make_uint4(0u, 0u, 0u, 0u);

            // ---- load cursor: the next row to request
            int          lt     = sw;  // its tile (>= L: the stream has ended)
            int          l_left = 0;   // vectors of that tile not yet requested
            const uint4* l_src  = p.compressed;
            auto load_enter_tile = [&]() {  // positions the cursor on the first non-empty tile at or after lt
                while (lt < L) {
                    const int vb = offs[lt], ve = offs[lt + 1];
                    int       n  = ve - vb;
                    n            = n < 0 ? 0 : (n > kMaxTileVectors ? kMaxTileVectors : n);
                    if (n > 0) {
                        l_left = n;
                        l_src  = p.compressed + vb;
                        if (lane == 0) {  // pull a later tile of this warp from DRAM into L2 ahead of its register loads
                            const int t = lt + kPrefetchAhead * NSW;
                            if (t < L && offs[t + 1] > offs[t])
                                ptx::prefetch_l2_bulk(p.compressed + offs[t], static_cast<uint32_t>(offs[t + 1] - offs[t]) * 16u);
                        }
                        return;
                    }
                    lt += NSW;
                }
                l_left = 0;
            };
            load_enter_tile();

            // ---- scatter cursor: the row about to be written
            int      st     = sw;               // its tile
            int      s_idx  = sw % a_stages;    // that tile's stage ...
            uint32_t s_par  = static_cast<uint32_t>(sw / a_stages) & 1u;  // ... and which use of it
            int      s_left = 0;                // vectors of that tile not yet scattered
            bool     ok     = true;

            // prologue: the first CAP rows of the stream
#pragma unroll
            for (int q = 0; q < CAP; ++q) {
                if (lt < L) {
                    if (lane < l_left)
                        win[q] = ldg_stream16(l_src + lane);
                    l_src += 32;
                    l_left -= 32;
                    if (l_left <= 0) {
                        lt += NSW;
                        load_enter_tile();
                    }
                }
            }

            // Enters tile st: waits until its stage holds zeros; tiles without words are published at once.
            auto scatter_enter_tile = [&]() {
                while (st < L) {
                    ok = wait_bounded_warp(a_zero + 8u * s_idx, s_par, abort_flag, p.status);
                    if (!ok)
                        return;
                    int n = offs[st + 1] - offs[st];
                    n     = n < 0 ? 0 : (n > kMaxTileVectors ? kMaxTileVectors : n);
                    if (n > 0) {
                        s_left = n;
                        return;
                    }
#ifndef FLASHLLM_CONSUMER_FENCE
                    ptx::fence_proxy_async_smem();  // the janitor's zeros, observed through a_zero, reach the tensor core
#endif
                    if (lane == 0)
                        ptx::mbar_arrive(a_full + 8u * s_idx);  // an all-zero tile
                    st += NSW;
                    s_idx += NSW;
                    while (s_idx >= a_stages) {
                        s_idx -= a_stages;
                        s_par ^= 1u;
                    }
                }
            };
            scatter_enter_tile();

            while (ok && st < L) {
#pragma unroll
                for (int q = 0; q < CAP; ++q) {
                    if (!(ok && st < L))
                        break;
                    const uint32_t stage = a_base + static_cast<uint32_t>(s_idx) * kDenseTileBytes;
                    if (lane < s_left)
                        scatter_vector(stage, win[q]);
                    s_left -= 32;
                    const bool tile_done = s_left <= 0;
                    if (tile_done) {
#ifndef FLASHLLM_CONSUMER_FENCE
                        ptx::fence_proxy_async_smem();  // generic-proxy stores -> the tensor core's async-proxy reads
#endif
                        __syncwarp();  // every lane's stores precede lane 0's release
                        if (lane == 0)
                            ptx::mbar_arrive(a_full + 8u * s_idx);
                    }
                    // the register is free again: request the row CAP places further down the stream
                    if (lt < L) {
                        if (lane < l_left)
                            win[q] = ldg_stream16(l_src + lane);
                        l_src += 32;
                        l_left -= 32;
                        if (l_left <= 0) {
                            lt += NSW;
                            load_enter_tile();
                        }
                    }
                    if (tile_done) {
                        st += NSW;
                        s_idx += NSW;
                        while (s_idx >= a_stages) {
                            s_idx -= a_stages;
                            s_par ^= 1u;
                        }
                        scatter_enter_tile();
                    }
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
    if (warp == mma_warp) {
        __syncwarp();
        ptx::tmem_dealloc(tmem_acc, kTmemCols);
    }
}

}  // namespace flashllm
