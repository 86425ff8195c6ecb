// Throughput of scattered shared-memory stores per SM: u16 vs u32 vs f16x2 reductions; conflict-free vs random banks.
#include <cstdio>
#include <cstdlib>
#include <cuda_runtime.h>
#include <cstdint>
#define CK(x) do { cudaError_t e = (x); if (e != cudaSuccess) { printf("ERR %s line %d: %s\n", #x, __LINE__, cudaGetErrorString(e)); exit(1);} } while (0)

template<int MODE>
__device__ __forceinline__ void op(uint32_t addr, uint32_t v)
{
    if (MODE == 0) asm volatile("st.shared.u16 [%0], %1;" ::"r"(addr), "h"((unsigned short)v) : "memory");
    if (MODE == 1) asm volatile("st.shared.u32 [%0], %1;" ::"r"(addr & ~3u), "r"(v) : "memory");
    if (MODE == 2) asm volatile("red.shared.add.noftz.f16x2 [%0], %1;" ::"r"(addr & ~3u), "r"(v) : "memory");
    if (MODE == 3) asm volatile("st.shared.u8 [%0], %1;" ::"r"(addr), "r"(v) : "memory");
}

// each warp owns 16 KB; 16 addresses per lane precomputed; `conflict`=0: lane l store i hits bank (l+5i)%32
template<int MODE>
__global__ void k(int reps, int conflict, long long* out)
{
    extern __shared__ __align__(16) unsigned char sm[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t base = (uint32_t)__cvta_generic_to_shared(sm) + warp * 16384;
    uint32_t a[16];
    uint32_t h = (blockIdx.x * 977 + threadIdx.x) * 2654435761u + 12345u;
    for (int i = 0; i < 16; ++i) {
        h = h * 1664525u + 1013904223u;
        const uint32_t row = (h >> 8) & 127u;          // 128 rows of 128 bytes
        uint32_t bank = conflict ? ((h >> 20) & 31u) : ((lane + 5 * i) & 31u);
        const uint32_t half = (h >> 27) & 1u;
        a[i] = base + row * 128u + bank * 4u + half * 2u;
    }
    for (int i = threadIdx.x; i < blockDim.x / 32 * 4096; i += blockDim.x) reinterpret_cast<uint32_t*>(sm)[i] = 0;
    __syncthreads();
    const long long t0 = clock64();
    for (int r = 0; r < reps; ++r) {
#pragma unroll
        for (int i = 0; i < 16; ++i) op<MODE>(a[i], 0x3C003C00u);
    }
    __syncthreads();
    const long long t1 = clock64();
    if (threadIdx.x == 0) out[blockIdx.x] = t1 - t0;
}

template<int MODE>
void run(const char* name, int warps, int conflict)
{
    long long* d; CK(cudaMalloc(&d, 148 * 8));
    const int smem = warps * 16384, reps = 2000;
    CK(cudaFuncSetAttribute(k<MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
    for (int it = 0; it < 2; ++it) { k<MODE><<<148, warps * 32, smem>>>(reps, conflict, d); CK(cudaDeviceSynchronize()); }
    long long h[148]; CK(cudaMemcpy(h, d, sizeof(h), cudaMemcpyDeviceToHost));
    double avg = 0; for (int i = 0; i < 148; ++i) avg += h[i]; avg /= 148;
    const double n = double(reps) * 16 * warps;
    printf("%-10s warps=%d conflict=%d : %.2f cycles per warp-store SM-wide (%.1f per warp)\n", name, warps, conflict, avg / n, avg / (double(reps) * 16));
    CK(cudaFree(d));
}

int main()
{
    for (int conflict = 0; conflict < 2; ++conflict)
        for (int warps : {1, 4, 8}) {
            run<0>("st.u16", warps, conflict);
            run<1>("st.u32", warps, conflict);
            run<2>("red.f16x2", warps, conflict);
            run<3>("st.u8", warps, conflict);
        }
    return 0;
}
