// Shared-memory contention between tcgen05.mma operand reads and LSU stores/loads: rates alone and together.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include "../../csrc/ptx_sm100.cuh"
using namespace flashllm;

// warp 0: MMA issuer (if do_mma). warps 1..W: store warps (mode 1: st.u16 scattered, 2: st.v4 zero-fill, 3: ld.shared.v4, 0: idle)
__global__ void __launch_bounds__(288, 1) k(int N, long long duration, int do_mma, int mode, int conflict, long long* out)
{
    extern __shared__ __align__(1024) uint8_t smem_raw[];
    const uint32_t base = (ptx::smem_u32(smem_raw) + 1023u) & ~1023u;
    __shared__ uint32_t tmem_slot;
    __shared__ __align__(8) unsigned long long bar;
    __shared__ long long counts[32];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int W = blockDim.x / 32 - 1;
    if (threadIdx.x == 0) { ptx::mbar_init(ptx::smem_u32(&bar), 1); ptx::fence_mbar_init(); }
    if (threadIdx.x < 32) counts[threadIdx.x] = 0;
    if (warp == 0) { ptx::tmem_alloc(ptx::smem_u32(&tmem_slot), 64); ptx::tmem_relinquish(); }
    // zero the whole dynamic region in use: (W + 2) * 16 KB
    for (uint32_t i = threadIdx.x; i < (uint32_t)(W + 2) * 4096u; i += blockDim.x)
        asm volatile("st.shared.u32 [%0], %1;" ::"r"(base + i * 4u), "r"(0u) : "memory");
    ptx::tc_fence_before_sync(); __syncthreads(); ptx::tc_fence_after_sync();
    const uint32_t tm = tmem_slot;
    const long long t0 = clock64();
    if (warp == 0) {
        if (lane == 0 && do_mma) {
            const uint32_t idesc = ptx::umma_idesc_f16_f32(128, N);
            const uint64_t da0 = ptx::umma_desc_kmajor_sw128(base), db0 = ptx::umma_desc_kmajor_sw128(base + 16384);
            long long n = 0;
            while (clock64() - t0 < duration) {
                for (int g = 0; g < 8; ++g) {
                    ptx::umma_f16_ss(tm, da0, db0, idesc, 1);
                    ptx::umma_f16_ss(tm, da0 + 2, db0 + 2, idesc, 1);
                    ptx::umma_f16_ss(tm, da0 + 4, db0 + 4, idesc, 1);
                    ptx::umma_f16_ss(tm, da0 + 6, db0 + 6, idesc, 1);
                }
                n += 32;
            }
            ptx::umma_commit(ptx::smem_u32(&bar));
            for (int spin = 0; spin < (1 << 24) && !ptx::mbar_test_wait(ptx::smem_u32(&bar), 0); ++spin) {}
            counts[0] = n;
            counts[20] = clock64() - t0;
        }
    }
    else if (mode != 0) {
        const uint32_t mine = base + (uint32_t)(warp + 1) * 16384u;
        uint32_t a[16];
        uint32_t h = (blockIdx.x * 977 + threadIdx.x) * 2654435761u + 12345u;
        for (int i = 0; i < 16; ++i) {
            h = h * 1664525u + 1013904223u;
            const uint32_t row = (h >> 8) & 127u;
            const uint32_t bank = conflict ? ((h >> 20) & 31u) : ((lane + 5 * i) & 31u);
            a[i] = mine + row * 128u + bank * 4u + ((h >> 27) & 1u) * 2u;
        }
        long long n = 0;
        uint32_t sink = 0;
        while (clock64() - t0 < duration) {
            if (mode == 1) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    asm volatile("st.shared.u16 [%0], %1;" ::"r"(a[i]), "h"((unsigned short)0x3C00) : "memory");
            }
            else if (mode == 4) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    asm volatile("st.shared.u32 [%0], %1;" ::"r"(a[i] & ~3u), "r"(0x3C003C00u) : "memory");
            }
            else if (mode == 5) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if ((lane + i) & 1)
                        asm volatile("st.shared.u16 [%0], %1;" ::"r"(a[i]), "h"((unsigned short)0x3C00) : "memory");
            }
            else if (mode == 6) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    if ((lane + i) & 1)
                        asm volatile("st.shared.u32 [%0], %1;" ::"r"(a[i] & ~3u), "r"(0x3C003C00u) : "memory");
            }
            else if (mode == 2) {
#pragma unroll
                for (int i = 0; i < 16; ++i)
                    asm volatile("st.shared.v4.b32 [%0], {%1, %1, %1, %1};" ::"r"(mine + (uint32_t)(i * 32 + lane) * 16u), "r"(0u) : "memory");
            }
            else {
#pragma unroll
                for (int i = 0; i < 16; ++i) {
                    uint32_t x, y, z, w;
                    asm volatile("ld.shared.v4.b32 {%0, %1, %2, %3}, [%4];" : "=r"(x), "=r"(y), "=r"(z), "=r"(w) : "r"(mine + (uint32_t)(i * 32 + lane) * 16u) : "memory");
                    sink ^= x ^ y ^ z ^ w;
                }
            }
            n += 16;
        }
        if (sink == 0x12345u) counts[31] = 1;
        if (lane == 0) { counts[warp] = n; }
    }
    __syncthreads();
    if (threadIdx.x < 32 && blockIdx.x == 0) out[threadIdx.x] = counts[threadIdx.x];
    if (warp == 0) { __syncwarp(); ptx::tmem_dealloc(tm, 64); }
}

int main()
{
    long long* d_out; cudaMalloc(&d_out, 32 * 8);
    cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
    const long long duration = 1000000;
    const char* names[] = {"idle", "st.u16 scattered", "st.v4 zero fill", "ld.v4", "st.u32 scattered", "st.u16 half lanes", "st.u32 half lanes"};
    for (int N : {16, 64})
        for (int W : {4, 8})
            for (int mode : {0, 1, 4, 5, 6, 2, 3})
                for (int conflict : {0, 1})
                    for (int do_mma : {0, 1}) {
                        if (mode == 0 && (!do_mma || conflict)) continue;
                        if (mode != 1 && mode != 4 && conflict) continue;
                        if (N == 64 && do_mma == 0) continue;
                        k<<<148, (W + 1) * 32, (W + 2) * 16384 + 1024>>>(N, duration, do_mma, mode, conflict, d_out);
                        cudaError_t e = cudaDeviceSynchronize();
                        long long h[32] = {0}; cudaMemcpy(h, d_out, sizeof(h), cudaMemcpyDeviceToHost);
                        long long ops = 0; for (int w = 1; w <= W; ++w) ops += h[w];
                        printf("N=%d W=%d lsu=%-17s conflict=%d mma=%d : ", N, W, names[mode], conflict, do_mma);
                        if (do_mma) printf("%.1f cycles/MMA ", (double)h[20] / (double)h[0]); else printf("                ");
                        if (mode) printf(" %.2f cycles per warp-LSU-op SM-wide", (double)duration / (double)ops);
                        printf(" %s\n", e ? cudaGetErrorString(e) : "");
                    }
    return 0;
}
