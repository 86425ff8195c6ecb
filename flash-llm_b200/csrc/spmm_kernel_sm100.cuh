// Load-as-Sparse / Compute-as-Dense SpMM for sm_100a.
//
// Does the work of the reference's SpMM_Kernel (csrc/SpMM_Kernel.cuh:179-386) and, for the K parts that live in one
// thread-block cluster, of SplitK_Reduction (csrc/Reduction_Kernel.cuh:24-45), with a different machine mapping:
//
//   * One CTA owns one 128-row tile row of A, one N tile of B and a contiguous range of 64-wide K tiles.  The
//     compressed words of that range are contiguous in Compressed_A, so a producer thread streams them as fixed-size
//     chunks with cp.async.bulk into a shared-memory ring, regardless of tile boundaries (the reference loads each
//     tile into registers with LDG.128, SpMM_Kernel.cuh:17-62).  The same thread fetches the [N_TILE x 64] B tiles
//     with TMA (128-byte swizzle), replacing the cp.async loader of MatMulUtilities.cuh:39-75.
//   * Scatter warps zero a dense 128x64 fp16 stage and write each word's value at its 16-bit location
//     (SpMM_Kernel.cuh:114-177 does the same from registers).  The location encoding r*64 + (c ^ ((r&7)<<3)) is
//     exactly the 128-byte-swizzled K-major layout tcgen05.mma reads, so reference-encoded buffers work unchanged.
//   * One thread issues four tcgen05.mma (M=128, N=N_TILE, K=16) per stage, accumulating fp32 in tensor memory
//     (replaces ldmatrix + mma.sync.m16n8k16, MatMulUtilities.cuh:77-132).
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
// 4 no MMA, 8 no ring reads, 16 no scatter-warp barrier.  Results are wrong with any bit set.
#ifndef FLASHLLM_ABLATE
#define FLASHLLM_ABLATE 0
#endif

// Spins on one mbarrier phase.  Returns false when the CTA has been told to give up, or after kWaitLimitNs,
// in which case it raises the abort flag and the status bit itself.
__device__ __forceinline__ bool
wait_bounded(uint32_t bar, uint32_t parity, volatile uint32_t* abort_flag, unsigned int* status)
{
    if (ptx::mbar_try_wait(bar, parity))
        return true;
    uint64_t t0 = 0;
    for (uint32_t it = 1;; ++it) {
        if (ptx::mbar_try_wait(bar, parity))
            return true;
        if ((it & 63u) == 0u) {
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

template<int N_TILE>
__global__ void __launch_bounds__(kMaxThreads, 1)
    spmm_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_b, const SpmmParams p)
{
    static_assert(N_TILE == 16 || N_TILE == 32 || N_TILE == 64 || N_TILE == 128, "unsupported MMA N");
    constexpr uint32_t kBBytes   = N_TILE * kTileK * 2;
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
    const int       ring_slots = plan.ring_slots;
    const int       CV         = plan.chunk_vectors;
    const int       S          = plan.cluster_k;
    const int       G          = plan.workspace_k;
    const int       NSW        = plan.scatter_warps;
    const int       NTS        = NSW * 32;

    // ---- shared memory carve-up
    const uint32_t a_base    = base;
    const uint32_t b_base    = a_base + a_stages * kDenseTileBytes;
    const uint32_t ring_base = b_base + b_stages * kBBytes;
    const uint32_t ring_vecs = ring_slots * CV;
    const uint32_t bar_base  = ring_base + ring_vecs * 16u;
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
    const int* const offs = p.tile_offsets + static_cast<long long>(tile_row) * p.k_tiles + k_begin;

    // ---- set-up
    if (threadIdx.x == 0) {
        // An earlier CTA that gave up leaves the status word set; later CTAs then skip their work.
        const unsigned int status_now = *reinterpret_cast<volatile unsigned int*>(p.status);
        for (int i = 0; i < ring_slots; ++i) {
            ptx::mbar_init(ring_full + 8u * i, 1);
            ptx::mbar_init(ring_empty + 8u * i, NSW);
        }
        for (int i = 0; i < a_stages; ++i) {
            ptx::mbar_init(a_full + 8u * i, NSW);
            ptx::mbar_init(a_empty + 8u * i, 1);
        }
        for (int i = 0; i < b_stages; ++i) {
            ptx::mbar_init(b_full + 8u * i, 1);
            ptx::mbar_init(b_empty + 8u * i, 1);
        }
        ptx::mbar_init(acc_full, 1);
        *abort_flag = (status_now != 0u) ? 1u : 0u;
        ptx::fence_mbar_init();
        ptx::prefetch_tensormap(&tmap_b);
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(const_cast<uint32_t*>(tmem_slot)), kTmemCols);
        ptx::tmem_relinquish();
    }
    ptx::tc_fence_before_sync();
    __syncthreads();
    ptx::tc_fence_after_sync();
    const uint32_t tmem_acc = *tmem_slot;

    if (warp == 0) {
        // ================================================================ producer: compressed stream + B tiles
        if (lane == 0 && L > 0) {
            const int v_first = offs[0];
            int       nvec    = offs[L] - v_first;
            if (nvec < 0)
                nvec = 0;  // the scatter warps report the malformed offsets
            const int    nchunks = (nvec + CV - 1) / CV;
            const uint4* src     = p.compressed + v_first;
            int          c = 0, c_slot = 0;
            uint32_t     c_use = 0;
            int          j = 0, j_slot = 0;
            uint32_t     j_use = 0;
            uint32_t     idle  = 0;
            uint64_t     t0    = 0;
            while (c < nchunks || j < L) {
                bool progressed = false;
                if (c < nchunks && ptx::mbar_test_wait(ring_empty + 8u * c_slot, (c_use & 1u) ^ 1u)) {
                    const int      left  = nvec - c * CV;
                    const uint32_t bytes = static_cast<uint32_t>(left < CV ? left : CV) * 16u;
                    const uint32_t bar   = ring_full + 8u * c_slot;
                    ptx::mbar_arrive_expect_tx(bar, bytes);
                    ptx::bulk_g2s(ring_base + static_cast<uint32_t>(c_slot) * CV * 16u, src + static_cast<size_t>(c) * CV,
                                  bytes, bar);
                    ++c;
                    if (++c_slot == ring_slots) {
                        c_slot = 0;
                        ++c_use;
                    }
                    progressed = true;
                }
                if (j < L && ptx::mbar_test_wait(b_empty + 8u * j_slot, (j_use & 1u) ^ 1u)) {
                    const uint32_t bar = b_full + 8u * j_slot;
                    ptx::mbar_arrive_expect_tx(bar, kBBytes);
                    ptx::tma_load_2d(b_base + j_slot * kBBytes, &tmap_b, (k_begin + j) * kTileK, n_idx * N_TILE, bar);
                    ++j;
                    if (++j_slot == b_stages) {
                        j_slot = 0;
                        ++j_use;
                    }
                    progressed = true;
                }
                if (progressed) {
                    idle = 0;
                }
                else if ((++idle & 1023u) == 0u) {
                    if (*abort_flag)
                        break;
                    const uint64_t now = ptx::globaltimer_ns();
                    if (idle == 1024u)
                        t0 = now;
                    else if (now - t0 > kWaitLimitNs) {
                        *abort_flag = 1u;
                        atomicOr(p.status, kStatusWaitExpired);
                        break;
                    }
                }
            }
            if (*abort_flag) {
                // Give copies already issued a bounded chance to land before the CTA may exit.
                const uint64_t t_leave = ptx::globaltimer_ns();
                for (int back = 1; back <= ring_slots && back <= c; ++back) {
                    const int      cc  = c - back;
                    const uint32_t bar = ring_full + 8u * (cc % ring_slots);
                    while (!ptx::mbar_try_wait(bar, (cc / ring_slots) & 1u)
                           && ptx::globaltimer_ns() - t_leave < 2000000ull) {}
                }
                for (int back = 1; back <= b_stages && back <= j; ++back) {
                    const int      jj  = j - back;
                    const uint32_t bar = b_full + 8u * (jj % b_stages);
                    while (!ptx::mbar_try_wait(bar, (jj / b_stages) & 1u)
                           && ptx::globaltimer_ns() - t_leave < 2000000ull) {}
                }
            }
        }
    }
    else if (warp == 1) {
        // ================================================================ MMA issuer
        if (lane == 0 && L > 0) {
            const uint32_t idesc  = ptx::umma_idesc_f16_f32(kTileM, N_TILE);
            int            s      = 0, bs = 0;
            uint32_t       a_use  = 0, b_use = 0;
            for (int j = 0; j < L; ++j) {
                if (!wait_bounded(a_full + 8u * s, a_use & 1u, abort_flag, p.status))
                    break;
                if (!wait_bounded(b_full + 8u * bs, b_use & 1u, abort_flag, p.status))
                    break;
                ptx::tc_fence_after_sync();
                const uint32_t a_addr = a_base + s * kDenseTileBytes;
                const uint32_t b_addr = b_base + bs * kBBytes;
#pragma unroll
                for (int kk = 0; kk < ((FLASHLLM_ABLATE & 4) ? 0 : kTileK / kUmmaK); ++kk) {
                    ptx::umma_f16_ss(tmem_acc,
                                     ptx::umma_desc_kmajor_sw128(a_addr + kk * kUmmaK * 2),
                                     ptx::umma_desc_kmajor_sw128(b_addr + kk * kUmmaK * 2),
                                     idesc,
                                     (j | kk) != 0 ? 1u : 0u);
                }
                ptx::umma_commit(a_empty + 8u * s);
                ptx::umma_commit(b_empty + 8u * bs);
                if (++s == a_stages) {
                    s = 0;
                    ++a_use;
                }
                if (++bs == b_stages) {
                    bs = 0;
                    ++b_use;
                }
            }
            ptx::umma_commit(acc_full);
        }
    }
    else {
        // ================================================================ scatter warps
        const int tid_s = threadIdx.x - kControlWarps * 32;
        if (L > 0) {
            // This CTA's slice of TileOffsets is read once, together, instead of one dependent load per tile.
            const int* offs_local = offs;
            if (L + 1 <= plan.offsets_staged) {
                for (int i = tid_s; i <= L; i += NTS)
                    offs_stage[i] = offs[i];
                ptx::named_barrier_sync(1, NTS);
                offs_local = offs_stage;
            }
            const int v_first  = offs_local[0];
            int       next_off = offs_local[1];
            int       vb       = 0;  // first vector of the current tile, relative to v_first
            int       ready    = 0;  // ring chunks known to have landed
            int       ready_slot = 0;
            uint32_t  ready_use  = 0;
            int       released = 0;  // ring chunks this warp has handed back
            int       rel_slot = 0;
            int       s        = 0;
            uint32_t  a_use    = 0;
            const int cv_shift = 31 - __clz(CV);
            for (int j = 0; j < L; ++j) {
                const int ve = next_off - v_first;
                if (j + 1 < L)
                    next_off = offs_local[j + 2];
                bool bad = (ve < vb) || (ve - vb > kMaxTileVectors);
                if (bad)
                    atomicOr(p.status, kStatusBadTileOffsets);
                const uint32_t stage = a_base + s * kDenseTileBytes;
                bool           ok    = !bad && wait_bounded(a_empty + 8u * s, (a_use & 1u) ^ 1u, abort_flag, p.status);
                if (ok) {
                    const int need = (ve + CV - 1) >> cv_shift;
                    while (ready < need) {
                        if (!wait_bounded(ring_full + 8u * ready_slot, ready_use & 1u, abort_flag, p.status)) {
                            ok = false;
                            break;
                        }
                        ++ready;
                        if (++ready_slot == ring_slots) {
                            ready_slot = 0;
                            ++ready_use;
                        }
                    }
                }
                if (ok && !(FLASHLLM_ABLATE & 1)) {
                    for (uint32_t off = tid_s * 16u; off < kDenseTileBytes; off += NTS * 16u)
                        sts_zero16(stage + off);
                }
                // Zeroes must be in place before any warp scatters; the same barrier makes giving up unanimous.
#if (FLASHLLM_ABLATE & 16)
                if (!ok || *abort_flag != 0u)
                    break;
#else
                if (barrier_any(1, NTS, !ok || *abort_flag != 0u)) {
                    if (bad)
                        *abort_flag = 1u;
                    break;
                }
#endif
                int      v   = vb + tid_s;
                uint32_t pos = static_cast<uint32_t>(v) % ring_vecs;
#if !(FLASHLLM_ABLATE & 8)
                for (; v < ve; v += NTS) {
                    const uint4 w = lds16(ring_base + pos * 16u);
#if (FLASHLLM_ABLATE & 2)
                    if ((w.x ^ w.y ^ w.z ^ w.w) == 0x9E3779B9u)  // keeps the loads alive; practically never true
                        scatter_word(stage, w.x);
#else
                    scatter_word(stage, w.x);
                    scatter_word(stage, w.y);
                    scatter_word(stage, w.z);
                    scatter_word(stage, w.w);
#endif
                    pos += NTS;
                    if (pos >= ring_vecs)
                        pos -= ring_vecs;
                }
#endif
                ptx::fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    const int done = ve >> cv_shift;  // chunks that end at or before this tile's last vector
                    while (released < done) {
                        ptx::mbar_arrive(ring_empty + 8u * rel_slot);
                        ++released;
                        if (++rel_slot == ring_slots)
                            rel_slot = 0;
                    }
                    ptx::mbar_arrive(a_full + 8u * s);
                }
                vb = ve;
                if (++s == a_stages) {
                    s = 0;
                    ++a_use;
                }
            }
        }

        // ================================================================ epilogue (same warps)
        bool acc_ok = true;
        if (L > 0)
            acc_ok = wait_bounded(acc_full, 0u, abort_flag, p.status);
        acc_ok = __all_sync(0xFFFFFFFFu, acc_ok && (*abort_flag == 0u));
        ptx::tc_fence_after_sync();

        const int quarter       = warp & 3;                 // TMEM lanes this warp may read: 32*quarter ..
        const int per_quarter   = NSW / 4;                  // warps sharing a lane quarter split the columns
        const int col_share     = (N_TILE / per_quarter) < 8 ? 8 : (N_TILE / per_quarter);
        const int col_begin     = ((warp - kControlWarps) / 4) * col_share;
        const int col_end       = (col_begin + col_share) < N_TILE ? (col_begin + col_share) : N_TILE;
        const int n_valid       = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
        const int row_in_tile   = quarter * 32 + lane;
        const size_t tile_off   = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
        half* const  out_tile   = p.out + tile_off;
        float* const part_tile  = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
        float* const red        = reinterpret_cast<float*>(smem);  // [N_TILE][128] fp32, over the idle A stages

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
        if (warp >= kControlWarps) {
            const int      tid_s    = threadIdx.x - kControlWarps * 32;
            const int      n_valid  = (p.N - n_idx * N_TILE) < N_TILE ? (p.N - n_idx * N_TILE) : N_TILE;
            const int      total    = N_TILE * kTileM;
            const int      lo       = static_cast<int>(static_cast<long long>(total) * rank / S);
            const int      hi       = static_cast<int>(static_cast<long long>(total) * (rank + 1) / S);
            const bool     store_ok = (*abort_flag == 0u);
            const size_t   tile_off = static_cast<size_t>(n_idx) * N_TILE * p.M + static_cast<size_t>(tile_row) * kTileM;
            half* const    out_tile = p.out + tile_off;
            float* const   part_tile = G > 1 ? p.partial + static_cast<size_t>(g) * p.M * p.N + tile_off : nullptr;
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
    if (warp == 1) {
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
