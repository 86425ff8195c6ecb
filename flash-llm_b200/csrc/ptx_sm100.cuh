// Thin inline-PTX wrappers for the sm_100a features the SpMM kernel uses: mbarrier, bulk async copies (TMA),
// tcgen05 tensor-core MMA with TMEM accumulators, proxy fences and thread-block-cluster shared memory.
// They take the place of the reference's mma.sync / ldmatrix / cp.async wrappers
// (csrc/MMA_PTX.cuh:15-98, csrc/AsyncCopy_PTX.cuh:15-78).
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace flashllm {
namespace ptx {

__device__ __forceinline__ uint32_t smem_u32(const void* p)
{
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// Flag traffic between GPUs: an acquire load at system scope (what it returns, and everything the writer did before
// its release, is visible to the loads that follow) and the matching release store.
__device__ __forceinline__ uint32_t ld_acquire_sys_u32(const unsigned int* ptr)
{
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

__device__ __forceinline__ uint32_t ld_relaxed_sys_u32(const unsigned int* ptr)
{
    uint32_t v;
    asm volatile("ld.relaxed.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(ptr) : "memory");
    return v;
}

__device__ __forceinline__ uint64_t globaltimer_ns()
{
    uint64_t t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

// ---------------------------------------------------------------- mbarrier

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void fence_mbar_init()
{
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

__device__ __forceinline__ void mbar_arrive(uint32_t bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}

// Arrival that counts as `count` pending arrivals at once.
__device__ __forceinline__ void mbar_arrive_count(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}

__device__ __forceinline__ void mbar_arrive_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}

// One probe of the phase with the given parity; true once that phase has completed.
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// Non-blocking probe of the phase with the given parity (try_wait may suspend the thread for a while).
__device__ __forceinline__ bool mbar_test_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n"
        "selp.u32 %0, 1, 0, p;\n"
        "}\n"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}

// ---------------------------------------------------------------- async copies

// 1-D bulk copy global -> this CTA's shared memory; size and both addresses are multiples of 16 bytes.
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

// 2-D tiled TMA load of one box (no multicast) into this CTA's shared memory.
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, int x, int y, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];" ::
            "r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(bar)
        : "memory");
}

// 3-D tiled TMA load of one box (no multicast) into this CTA's shared memory.
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, int x, int y, int z, uint32_t bar)
{
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];" ::
            "r"(dst),
        "l"(map), "r"(x), "r"(y), "r"(z), "r"(bar)
        : "memory");
}

// Asks the memory system to bring [src, src + bytes) into L2 (16-byte aligned address, size a multiple of 16); no
// completion is signalled and nothing is written to shared memory or registers.
__device__ __forceinline__ void prefetch_l2_bulk(const void* src, uint32_t bytes)
{
    asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(src), "r"(bytes) : "memory");
}

__device__ __forceinline__ void prefetch_tensormap(const CUtensorMap* map)
{
    asm volatile("prefetch.tensormap [%0];" ::"l"(map) : "memory");
}

// Makes this thread's earlier generic-proxy shared-memory writes visible to the async proxy (UMMA, TMA).
__device__ __forceinline__ void fence_proxy_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}

// ---------------------------------------------------------------- tcgen05 / TMEM

__device__ __forceinline__ void tmem_alloc(uint32_t smem_result, uint32_t ncols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_result), "r"(ncols)
                 : "memory");
}

__device__ __forceinline__ void tmem_relinquish()
{
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}

__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}

__device__ __forceinline__ void tc_fence_before_sync()
{
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}

__device__ __forceinline__ void tc_fence_after_sync()
{
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}

// D[tmem] (+)= A[smem] * B[smem], fp16 inputs, fp32 accumulate, issued by one thread for the CTA.
__device__ __forceinline__ void
umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
        : "memory");
}

// One 128x64 tile of A times one [N x 64] slab of B: the four K=16 MMAs, the commit that hands the A stage back, an
// optional second commit (B batch finished), and -- issued first so that its shared-memory round trip overlaps the
// MMA issue -- a probe of the barriers the NEXT tile needs.  All in one asm block because the probe's predicate must
// survive until after the MMAs, which separate asm statements cannot express.  Returns whether the next tile's
// barriers had completed at probe time.
__device__ __forceinline__ bool umma_tile_commit_probe(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                                       uint32_t accumulate_first, uint32_t commit_a_bar,
                                                       uint32_t commit_b_bar, uint32_t do_commit_b,
                                                       uint32_t next_a_bar, uint32_t next_a_par, uint32_t next_b_bar,
                                                       uint32_t next_b_par, uint32_t probe_a, uint32_t probe_b)
{
    uint32_t ready;
    asm volatile(
        "{\n"
        ".reg .pred pacc, ptrue, pna, pnb, pda, pdb, pcb;\n"
        ".reg .b64 da, db;\n"
        "setp.ne.b32 pacc, %5, 0;\n"
        "setp.eq.b32 ptrue, 0, 0;\n"
        "setp.ne.b32 pda, %13, 0;\n"
        "setp.ne.b32 pdb, %14, 0;\n"
        "setp.ne.b32 pcb, %8, 0;\n"
        "setp.eq.b32 pna, 0, 0;\n"
        "setp.eq.b32 pnb, 0, 0;\n"
        "@pda mbarrier.test_wait.parity.shared::cta.b64 pna, [%9], %10;\n"
        "@pdb mbarrier.test_wait.parity.shared::cta.b64 pnb, [%11], %12;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], %2, %3, %4, pacc;\n"
        "add.s64 da, %2, 2;\n"
        "add.s64 db, %3, 2;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %4, ptrue;\n"
        "add.s64 da, %2, 4;\n"
        "add.s64 db, %3, 4;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %4, ptrue;\n"
        "add.s64 da, %2, 6;\n"
        "add.s64 db, %3, 6;\n"
        "tcgen05.mma.cta_group::1.kind::f16 [%1], da, db, %4, ptrue;\n"
        "tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%6];\n"
        "@pcb tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%7];\n"
        "and.pred pna, pna, pnb;\n"
        "selp.u32 %0, 1, 0, pna;\n"
        "}\n"
        : "=r"(ready)
        : "r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate_first), "r"(commit_a_bar), "r"(commit_b_bar),
          "r"(do_commit_b), "r"(next_a_bar), "r"(next_a_par), "r"(next_b_bar), "r"(next_b_par), "r"(probe_a),
          "r"(probe_b)
        : "memory");
    return ready != 0;
}

// Arrives once on the mbarrier when every tcgen05 operation issued so far by this thread has completed.
__device__ __forceinline__ void umma_commit(uint32_t bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}

// Each thread reads 8 consecutive fp32 columns of its own TMEM lane (lane = 32*(warp%4) + laneid).
__device__ __forceinline__ void tmem_ld_x8(uint32_t taddr, uint32_t (&r)[8])
{
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
                 : "r"(taddr)
                 : "memory");
}

__device__ __forceinline__ void tmem_wait_ld()
{
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Shared-memory matrix descriptor of a K-major operand whose rows are 128 bytes (64 fp16), stored with the
// 128-byte swizzle in groups of 8 rows (1024 bytes per group); `addr` is the 1024-byte-aligned tile base
// plus 32 bytes per 16-wide K step.
__device__ __forceinline__ uint64_t umma_desc_kmajor_sw128(uint32_t addr)
{
    uint64_t d = 0;
    d |= static_cast<uint64_t>((addr & 0x3FFFFu) >> 4);  // start address, 16-byte units
    d |= static_cast<uint64_t>(1) << 16;                 // leading byte offset: unused with swizzled K-major
    d |= static_cast<uint64_t>(1024 >> 4) << 32;         // stride byte offset: next 8-row group
    d |= static_cast<uint64_t>(1) << 46;                 // descriptor version for sm_100
    d |= static_cast<uint64_t>(2) << 61;                 // layout: 128-byte swizzle
    return d;
}

// Instruction descriptor for kind::f16: fp16 A and B (both K-major), fp32 D, M x N tile.
__device__ __forceinline__ uint32_t umma_idesc_f16_f32(uint32_t m, uint32_t n)
{
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// ---------------------------------------------------------------- programmatic dependent launch

// Lets the next kernel of the stream (if it was launched with the programmatic-serialisation attribute) start its
// CTAs as soon as every CTA of this grid has executed this or exited.
__device__ __forceinline__ void grid_launch_dependents()
{
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
}

// Blocks until every kernel this one depends on has completed and its writes are visible; returns at once for a
// kernel that was launched without the attribute.
__device__ __forceinline__ void grid_dependency_wait()
{
    asm volatile("griddepcontrol.wait;" ::: "memory");
}

// ---------------------------------------------------------------- cluster

__device__ __forceinline__ uint32_t cluster_ctarank()
{
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}

__device__ __forceinline__ void cluster_sync_all()
{
    asm volatile("barrier.cluster.arrive.release.aligned;\n"
                 "barrier.cluster.wait.acquire.aligned;\n" ::
                     : "memory");
}

// Address of the same shared-memory location in the CTA of the given cluster rank.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local_addr, uint32_t rank)
{
    uint32_t remote;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(remote) : "r"(local_addr), "r"(rank));
    return remote;
}

__device__ __forceinline__ float ld_dsmem_f32(uint32_t addr)
{
    float v;
    asm volatile("ld.shared::cluster.f32 %0, [%1];" : "=f"(v) : "r"(addr) : "memory");
    return v;
}

__device__ __forceinline__ float4 ld_dsmem_v4_f32(uint32_t addr)
{
    float4 v;
    asm volatile("ld.shared::cluster.v4.f32 {%0, %1, %2, %3}, [%4];"
                 : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                 : "r"(addr)
                 : "memory");
    return v;
}

__device__ __forceinline__ void named_barrier_sync(uint32_t id, uint32_t threads)
{
    asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory");
}

}  // namespace ptx
}  // namespace flashllm
