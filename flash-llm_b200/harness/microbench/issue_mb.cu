// Cost per tile of the MMA issuer's instruction sequence on an otherwise idle SM: 4 MMAs, commits, barrier probes.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include "../../csrc/ptx_sm100.cuh"
using namespace flashllm;

__global__ void __launch_bounds__(64, 1) k(int N, int tiles, int mode, long long* out)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bars[16];
    const int warp = threadIdx.x >> 5;
    if (threadIdx.x == 0) { for (int i = 0; i < 16; ++i) ptx::mbar_init(ptx::smem_u32(&bars[i]), 1); ptx::fence_mbar_init(); }
    if (warp == 0) { ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 64); ptx::tmem_relinquish(); }
    for (uint32_t i = threadIdx.x; i < 5u * 4096u; i += blockDim.x)
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + i * 4u), "r"(0u) : "memory");
    ptx::tc_fence_before_sync(); __syncthreads(); ptx::tc_fence_after_sync();
    const uint32_t tm = tmem_slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = ptx::umma_idesc_f16_f32(128, N);
        const uint64_t da0 = ptx::umma_desc_kmajor_sw128(base), db0 = ptx::umma_desc_kmajor_sw128(base + 4 * 16384);
        const uint32_t b0 = ptx::smem_u32(&bars[0]);
        const long long t0 = clock64();
        uint32_t ready_acc = 0;
        for (int j = 0; j < tiles; ++j) {
            const int s = j & 3;
            const uint64_t da = da0 + (uint32_t)(s * 1024);
            if (mode == 0 || mode == 1 || mode == 2) {
                ptx::umma_f16_ss(tm, da, db0, idesc, 1);
                ptx::umma_f16_ss(tm, da + 2, db0 + 2, idesc, 1);
                ptx::umma_f16_ss(tm, da + 4, db0 + 4, idesc, 1);
                ptx::umma_f16_ss(tm, da + 6, db0 + 6, idesc, 1);
                if (mode >= 1) ptx::umma_commit(b0 + 8u * s);
                if (mode >= 2) ptx::umma_commit(b0 + 8u * (4 + (j & 1)));
            }
            else if (mode == 3) {   // the kernel's fused block, probing barriers 8.. that never complete parity 1 -> returns not ready
                ready_acc += ptx::umma_tile_commit_probe(tm, da, db0, idesc, 1u, b0 + 8u * s, b0 + 8u * (4 + (j & 1)), (j & 1), b0 + 8u * 8, 1u,
                                                         b0 + 8u * 9, 1u, 1u, (j & 1));
            }
            else if (mode == 4) {   // fence + fused block as in the kernel loop
                ptx::tc_fence_after_sync();
                ready_acc += ptx::umma_tile_commit_probe(tm, da, db0, idesc, 1u, b0 + 8u * s, b0 + 8u * (4 + (j & 1)), (j & 1), b0 + 8u * 8, 1u,
                                                         b0 + 8u * 9, 1u, 1u, (j & 1));
            }
        }
        const long long t1 = clock64();
        ptx::umma_commit(b0 + 8u * 10);
        for (int spin = 0; spin < (1 << 24) && !ptx::mbar_test_wait(b0 + 8u * 10, 0); ++spin) {}
        const long long t2 = clock64();
        if (blockIdx.x == 0) { out[0] = t1 - t0; out[1] = t2 - t0; out[2] = ready_acc; }
    }
    __syncthreads();
    if (warp == 0) { __syncwarp(); ptx::tmem_dealloc(tm, 64); }
}

int main()
{
    long long* d_out; cudaMalloc(&d_out, 32);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 100 * 1024);
    const int tiles = 4000;
    const char* names[] = {"4 MMA", "4 MMA + commit", "4 MMA + 2 commits", "fused block (probes+4 MMA+commits)", "fence + fused block"};
    for (int N : {16, 64})
        for (int mode = 0; mode < 5; ++mode) {
            k<<<148, 64, 6 * 16384>>>(N, tiles, mode, d_out);
            k<<<148, 64, 6 * 16384>>>(N, tiles, mode, d_out);
            cudaError_t e = cudaDeviceSynchronize();
            long long h[3] = {0}; cudaMemcpy(h, d_out, 24, cudaMemcpyDeviceToHost);
            printf("N=%d %-36s: issue %.1f cycles per tile, to completion %.1f %s\n", N, names[mode], (double)h[0] / tiles, (double)h[1] / tiles, e ? cudaGetErrorString(e) : "");
        }
    return 0;
}
