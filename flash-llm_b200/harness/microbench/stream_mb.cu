// Microbenchmark: HBM read streaming rates on B200 for (a) cp.async.bulk into a smem ring, (b) LDG.128 grid-stride.
#include <cuda_runtime.h>
#include <cstdio>
#include <cstdint>
#include <cstdlib>
#include <vector>

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t c) { asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(c) : "memory"); }
__device__ __forceinline__ void mbar_expect(uint32_t bar, uint32_t b) { asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(b) : "memory"); }
__device__ __forceinline__ bool mbar_try(uint32_t bar, uint32_t ph) { uint32_t ok; asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0,1,0,p;\n}\n" : "=r"(ok) : "r"(bar), "r"(ph) : "memory"); return ok; }
__device__ __forceinline__ void bulk(uint32_t dst, const void* src, uint32_t bytes, uint32_t bar) { asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst), "l"(src), "r"(bytes), "r"(bar) : "memory"); }

// One thread per CTA: keeps `slots` copies of `chunk` bytes in flight over its contiguous region; consumption = wait.
// mode 0: single thread does both issue+wait (slot reuse right after completion).
__global__ void ring_stream_multi(const uint8_t* src, size_t bytes_per_thread, int chunk, int slots, int producers, int tstride, unsigned long long* sink)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t ring0 = smem_u32(smem);
    const uint32_t bars0 = ring0 + (uint32_t)chunk * slots * producers;
    if (threadIdx.x == 0) {
        for (int i = 0; i < slots * producers; ++i) mbar_init(bars0 + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x % tstride == 0 && threadIdx.x / tstride < producers) {
        const int p = threadIdx.x / tstride;
        const uint32_t ring = ring0 + p * chunk * slots;
        const uint32_t bars = bars0 + 8 * p * slots;
        const uint8_t* base = src + ((size_t)blockIdx.x * producers + p) * bytes_per_thread;
        const long long n = (long long)(bytes_per_thread / chunk);
        long long issued = 0, done = 0;
        unsigned long long acc = 0;
        long long spins = 0;
        while (done < n) {
            while (issued < n && issued - done < slots) {
                const int s = (int)(issued % slots);
                mbar_expect(bars + 8 * s, chunk);
                bulk(ring + s * chunk, base + issued * (size_t)chunk, chunk, bars + 8 * s);
                ++issued;
            }
            const int s = (int)(done % slots);
            const uint32_t ph = (uint32_t)((done / slots) & 1);
            while (!mbar_try(bars + 8 * s, ph)) { if (++spins > (1ll << 26)) { done = n; break; } }
            ++done;
        }
        if (acc == 0x1234567ull) *sink = acc;
    }
}

__global__ void ring_stream(const uint8_t* src, size_t bytes_per_cta, int chunk, int slots, unsigned long long* sink)
{
    extern __shared__ __align__(1024) uint8_t smem[];
    const uint32_t ring = smem_u32(smem);
    const uint32_t bars = ring + (uint32_t)chunk * slots;
    if (threadIdx.x == 0) {
        for (int i = 0; i < slots; ++i) mbar_init(bars + 8 * i, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        const uint8_t* base = src + (size_t)blockIdx.x * bytes_per_cta;
        const long long n = (long long)(bytes_per_cta / chunk);
        long long issued = 0, done = 0;
        unsigned long long acc = 0;
        long long spins = 0;
        while (done < n) {
            while (issued < n && issued - done < slots) {
                const int s = (int)(issued % slots);
                mbar_expect(bars + 8 * s, chunk);
                bulk(ring + s * chunk, base + issued * (size_t)chunk, chunk, bars + 8 * s);
                ++issued;
            }
            const int s = (int)(done % slots);
            const uint32_t ph = (uint32_t)((done / slots) & 1);
            while (!mbar_try(bars + 8 * s, ph)) { if (++spins > (1ll << 26)) { done = n; break; } }
            acc += *(volatile uint32_t*)(smem + s * chunk);
            ++done;
        }
        if (acc == 0x1234567ull) *sink = acc;
    }
}

__global__ void ldg_stream(const uint4* src, size_t vecs, unsigned long long* sink)
{
    size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    uint32_t acc = 0;
    for (; i + 3 * stride < vecs; i += 4 * stride) {
        uint4 a = __ldg(src + i), b = __ldg(src + i + stride), c = __ldg(src + i + 2 * stride), d = __ldg(src + i + 3 * stride);
        acc ^= a.x ^ b.y ^ c.z ^ d.w;
    }
    if (acc == 0x12345u) *sink = acc;
}

// Per-CTA contiguous LDG (each CTA reads its own contiguous region, like the SpMM does)
__global__ void ldg_stream_cta(const uint4* src, size_t vecs_per_cta, unsigned long long* sink)
{
    const uint4* base = src + (size_t)blockIdx.x * vecs_per_cta;
    uint32_t acc = 0;
    for (size_t i = threadIdx.x; i + 3 * blockDim.x < vecs_per_cta; i += 4 * blockDim.x) {
        uint4 a = __ldg(base + i), b = __ldg(base + i + blockDim.x), c = __ldg(base + i + 2 * blockDim.x), d = __ldg(base + i + 3 * blockDim.x);
        acc ^= a.x ^ b.y ^ c.z ^ d.w;
    }
    if (acc == 0x12345u) *sink = acc;
}

int main()
{
    const size_t total = (size_t)2 << 30;  // 2 GiB
    uint8_t* buf; cudaMalloc(&buf, total); cudaMemset(buf, 1, total);
    unsigned long long* sink; cudaMalloc(&sink, 8);
    cudaEvent_t e0, e1; cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaFuncSetAttribute(ring_stream, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    int sms = 148;
    auto run_ring = [&](int ctas, int chunk, int slots) {
        size_t per = (total / ctas) / chunk * chunk;
        size_t smem = (size_t)chunk * slots + 8 * slots + 64;
        if (smem > 227 * 1024) return;
        float best = 1e9;
        for (int r = 0; r < 3; ++r) {
            cudaEventRecord(e0);
            ring_stream<<<ctas, 32, smem>>>(buf, per, chunk, slots, sink);
            cudaEventRecord(e1); cudaEventSynchronize(e1);
            float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
        }
        cudaError_t err = cudaGetLastError();
        printf("ring ctas=%d (%.1f/SM) chunk=%d slots=%d inflight/CTA=%dKB: %.0f GB/s %s\n", ctas, (double)ctas / sms, chunk, slots,
               chunk * slots / 1024, (double)per * ctas / best / 1e6, err ? cudaGetErrorString(err) : "");
    };
    cudaFuncSetAttribute(ring_stream_multi, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    auto run_multi = [&](int ctas, int chunk, int slots, int producers, int tstride) {
        size_t per = (total / ctas / producers) / chunk * chunk;
        size_t smem = (size_t)chunk * slots * producers + 8 * slots * producers + 64;
        if (smem > 227 * 1024) return;
        float best = 1e9;
        for (int r = 0; r < 3; ++r) {
            cudaEventRecord(e0);
            ring_stream_multi<<<ctas, 1024, smem>>>(buf, per, chunk, slots, producers, tstride, sink);
            cudaEventRecord(e1); cudaEventSynchronize(e1);
            float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
        }
        cudaError_t err = cudaGetLastError();
        printf("multi ctas=%d chunk=%d slots=%d producers=%d tstride=%d: %.0f GB/s %s\n", ctas, chunk, slots, producers, tstride,
               (double)per * ctas * producers / best / 1e6, err ? cudaGetErrorString(err) : "");
    };
    for (int chunk : {1024, 4096})
        for (int producers : {1, 2, 4, 8, 16})
            for (int tstride : {1, 32}) run_multi(148, chunk, 4, producers, tstride);
    for (int chunk : {8192, 32768, 65536})
        for (int slots : {2, 3, 4, 8}) run_ring(148, chunk, slots);
    for (int chunk : {2048, 8192})
        for (int slots : {4, 8}) run_ring(296, chunk, slots);
    for (int threads : {1024})
        for (int ctas : {148 * 2}) {
            float best = 1e9;
            for (int r = 0; r < 3; ++r) {
                cudaEventRecord(e0);
                ldg_stream<<<ctas, threads>>>((const uint4*)buf, total / 16, sink);
                cudaEventRecord(e1); cudaEventSynchronize(e1);
                float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
            }
            printf("ldg grid-stride ctas=%d threads=%d: %.0f GB/s\n", ctas, threads, (double)total / best / 1e6);
            best = 1e9;
            for (int r = 0; r < 3; ++r) {
                cudaEventRecord(e0);
                ldg_stream_cta<<<ctas, threads>>>((const uint4*)buf, total / 16 / ctas, sink);
                cudaEventRecord(e1); cudaEventSynchronize(e1);
                float ms; cudaEventElapsedTime(&ms, e0, e1); if (ms < best) best = ms;
            }
            printf("ldg per-CTA contiguous ctas=%d threads=%d: %.0f GB/s\n", ctas, threads, (double)total / best / 1e6);
        }
    return 0;
}
