// Benchmark and correctness driver for libSpMM_API.so with the command line of the reference's
// kernel_benchmark/spmm_test.cu (:47-55):   ./spmm_test M K N Sparsity(percent) SplitK [--ref libSpMM_API_ref.so]
//
// Inputs are seeded (counter-based splitmix64, the generator of flash-llm_b200/synthetic.py): A has a Bernoulli mask
// with the given sparsity and U(-1,1) non-zeros, B is U(-1,1).  A is encoded on the host (InitSparseMatrixA_API) and
// on the device (FlashLLM_EncodeOnDevice_*), the two encodings are compared bit for bit, the SpMM is timed with CUDA
// events (20 warm-up + 200 timed launches; the reference uses 100 + 10000, spmm_test_utils.h:21-22) and checked
// against a host fp32 GEMM with the reference's TotalError (spmm_test_utils.h:120-126) and a max relative error.
// With --ref, the unmodified reference library is loaded beside this one (dlopen, local symbols) and timed on the
// same device buffers.
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <thread>
#include <string>
#include <vector>

#include "../../include/SpMM_API.cuh"

#define CHECK_CUDA(x)                                                                                                  \
    do {                                                                                                               \
        cudaError_t e_ = (x);                                                                                          \
        if (e_ != cudaSuccess) {                                                                                       \
            printf("CUDA error %s at line %d\n", cudaGetErrorString(e_), __LINE__);                                    \
            exit(EXIT_FAILURE);                                                                                        \
        }                                                                                                              \
    } while (0)

static inline uint64_t mix(uint64_t z)
{
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ull;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBull;
    return z ^ (z >> 31);
}

static inline float uniform01(uint64_t seed, uint64_t index, uint64_t stream)
{
    const uint64_t z = mix((index + 1) * 0x9E3779B97F4A7C15ull + seed + stream * 0x632BE59BD9B4E019ull);
    return static_cast<float>(z >> 40) * (1.0f / 16777216.0f);
}

template<typename F>
static void parallel_rows(int rows, F&& body)
{
    unsigned n = std::thread::hardware_concurrency();
    if (n == 0)
        n = 1;
    std::vector<std::thread> pool;
    for (unsigned t = 0; t < n; ++t)
        pool.emplace_back([&, t]() {
            for (int r = static_cast<int>(t); r < rows; r += static_cast<int>(n))
                body(r);
        });
    for (auto& th : pool)
        th.join();
}

using SpmmFn = cudaError_t (*)(cudaStream_t, const half*, const uint4*, const int*, const half*, half*, int, int, int,
                               half*, int);

static float time_spmm(SpmmFn fn, const uint4* nz, const int* offs, const half* B, half* C, int M, int N, int K, half* ws,
                       int split_k, int warmup, int iters)
{
    cudaEvent_t start, stop;
    CHECK_CUDA(cudaEventCreate(&start));
    CHECK_CUDA(cudaEventCreate(&stop));
    for (int i = 0; i < warmup; ++i)
        CHECK_CUDA(fn(0, nullptr, nz, offs, B, C, M, N, K, ws, split_k));
    CHECK_CUDA(cudaEventRecord(start));
    for (int i = 0; i < iters; ++i)
        fn(0, nullptr, nz, offs, B, C, M, N, K, ws, split_k);
    CHECK_CUDA(cudaEventRecord(stop));
    CHECK_CUDA(cudaEventSynchronize(stop));
    CHECK_CUDA(cudaGetLastError());
    float ms = 0.f;
    CHECK_CUDA(cudaEventElapsedTime(&ms, start, stop));
    return ms / iters;
}

int main(int argc, char** argv)
{
    if (argc < 6) {
        printf("Wrong Inputs! Correct input format: ./spmm_test M K N Sparsity SplitK [--ref path/to/reference.so] [--plan name=value,...] [--overlap 0|1]\n");
        return 1;
    }
    const int   M = atoi(argv[1]), K = atoi(argv[2]), N = atoi(argv[3]), sparsity_pct = atoi(argv[4]), split_k = atoi(argv[5]);
    // optional, in any order after the five numbers: --ref <reference .so>, --overlap 0|1 (launch overlap of
    // consecutive SpMMs, off unless given), --plan name=value[,name=value...]
    // (the fields of FlashLLM_SetPlan: cluster_k, workspace_k, a_stages, b_stages, b_batch, ring_slots, chunk_vectors,
    // scatter_warps, producers, path, reduce)
    const char* ref_path = nullptr;
    for (int a = 6; a + 1 < argc; a += 2) {
        if (strcmp(argv[a], "--ref") == 0)
            ref_path = argv[a + 1];
        else if (strcmp(argv[a], "--plan") == 0) {
            static const char* names[11] = {"cluster_k",  "workspace_k",   "a_stages",      "b_stages",  "b_batch", "ring_slots",
                                            "chunk_vectors", "scatter_warps", "producers", "path", "reduce"};
            int                fields[11] = {0};
            std::string        spec(argv[a + 1]);
            size_t             pos = 0;
            while (pos < spec.size()) {
                const size_t end = spec.find(',', pos);
                const std::string item = spec.substr(pos, end == std::string::npos ? std::string::npos : end - pos);
                const size_t eq = item.find('=');
                bool known = false;
                for (int f = 0; f < 11 && eq != std::string::npos; ++f)
                    if (item.compare(0, eq, names[f]) == 0) {
                        fields[f] = atoi(item.c_str() + eq + 1);
                        known     = true;
                    }
                if (!known) {
                    printf("unknown plan field in '%s'\n", item.c_str());
                    return 1;
                }
                pos = end == std::string::npos ? spec.size() : end + 1;
            }
            FlashLLM_SetPlan(fields, 11);
        }
        else if (strcmp(argv[a], "--overlap") == 0)
            FlashLLM_SetLaunchOverlap(atoi(argv[a + 1]));
        else {
            printf("unknown option %s\n", argv[a]);
            return 1;
        }
    }
    const float sparsity = sparsity_pct / 100.0f;
    const uint64_t seed_a = 0xF1A50000ull + static_cast<uint64_t>(sparsity_pct), seed_b = seed_a ^ 0xB;

    std::vector<half> A_h(static_cast<size_t>(M) * K), B_h(static_cast<size_t>(N) * K);
    parallel_rows(M, [&](int r) {
        for (int c = 0; c < K; ++c) {
            const uint64_t i    = static_cast<uint64_t>(r) * K + c;
            const bool     keep = uniform01(seed_a, i, 0) >= sparsity;
            float          v    = uniform01(seed_a, i, 1) * 2.0f - 1.0f;
            if (fabsf(v) < 6.2e-5f)
                v = v < 0 ? -6.2e-5f : 6.2e-5f;
            A_h[i] = __float2half_rn(keep ? v : 0.0f);
        }
    });
    for (size_t i = 0; i < B_h.size(); ++i)
        B_h[i] = __float2half_rn(uniform01(seed_b, i, 2) * 2.0f - 1.0f);

    // ---- host encoder
    uint32_t* nz_h   = nullptr;
    int*      offs_h = nullptr;
    const int num_offsets = InitSparseMatrixA_API(A_h.data(), M, N, K, &nz_h, &offs_h);
    const int nnz         = offs_h[num_offsets - 1] * 4;

    half *A_d, *B_d, *C_d, *ws_d;
    int*      offs_d;
    uint32_t *nz_d, *nz_dev_encoded;
    CHECK_CUDA(cudaMalloc(&A_d, sizeof(half) * A_h.size()));
    CHECK_CUDA(cudaMalloc(&B_d, sizeof(half) * B_h.size()));
    CHECK_CUDA(cudaMalloc(&C_d, sizeof(half) * M * N));
    CHECK_CUDA(cudaMalloc(&ws_d, sizeof(half) * static_cast<size_t>(M) * N * (split_k > 0 ? split_k : 1)));
    CHECK_CUDA(cudaMalloc(&offs_d, sizeof(int) * num_offsets));
    CHECK_CUDA(cudaMalloc(&nz_d, sizeof(uint32_t) * (nnz > 0 ? nnz : 4)));
    CHECK_CUDA(cudaMalloc(&nz_dev_encoded, sizeof(uint32_t) * (nnz > 0 ? nnz : 4)));
    CHECK_CUDA(cudaMemcpy(A_d, A_h.data(), sizeof(half) * A_h.size(), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(B_d, B_h.data(), sizeof(half) * B_h.size(), cudaMemcpyHostToDevice));
    CHECK_CUDA(cudaMemcpy(nz_d, nz_h, sizeof(uint32_t) * nnz, cudaMemcpyHostToDevice));

    // ---- device encoder, checked against the host encoder
    cudaEvent_t e0, e1;
    CHECK_CUDA(cudaEventCreate(&e0));
    CHECK_CUDA(cudaEventCreate(&e1));
    CHECK_CUDA(cudaEventRecord(e0));
    CHECK_CUDA(static_cast<cudaError_t>(FlashLLM_EncodeOnDevice_TileOffsets(nullptr, A_d, M, K, offs_d)));
    CHECK_CUDA(static_cast<cudaError_t>(FlashLLM_EncodeOnDevice_Pack(nullptr, A_d, M, K, offs_d, nz_dev_encoded, 1)));
    CHECK_CUDA(cudaEventRecord(e1));
    CHECK_CUDA(cudaEventSynchronize(e1));
    float encode_ms = 0.f;
    CHECK_CUDA(cudaEventElapsedTime(&encode_ms, e0, e1));
    std::vector<int>      offs_back(num_offsets);
    std::vector<uint32_t> nz_back(nnz > 0 ? nnz : 1);
    CHECK_CUDA(cudaMemcpy(offs_back.data(), offs_d, sizeof(int) * num_offsets, cudaMemcpyDeviceToHost));
    CHECK_CUDA(cudaMemcpy(nz_back.data(), nz_dev_encoded, sizeof(uint32_t) * nnz, cudaMemcpyDeviceToHost));
    const bool encoders_agree = memcmp(offs_back.data(), offs_h, sizeof(int) * num_offsets) == 0
                                && memcmp(nz_back.data(), nz_h, sizeof(uint32_t) * nnz) == 0;

    // ---- SpMM
    printf("Launching Flash-LLM (B200 library)...\n");
    const float ms = time_spmm(SpMM_SplitK_API, reinterpret_cast<uint4*>(nz_d), offs_d, B_d, C_d, M, N, K, ws_d, split_k, 20, 200);
    std::vector<half> C_h(static_cast<size_t>(M) * N);
    CHECK_CUDA(cudaMemcpy(C_h.data(), C_d, sizeof(half) * C_h.size(), cudaMemcpyDeviceToHost));
    const unsigned status = FlashLLM_ConsumeStatus();

    // ---- host fp32 GEMM check: C[n][m] = sum_k A[m][k] * B[n][k]
    std::vector<float> want(static_cast<size_t>(M) * N), Bf(B_h.size());
    for (size_t i = 0; i < B_h.size(); ++i)
        Bf[i] = __half2float(B_h[i]);
    parallel_rows(M, [&](int m) {
        std::vector<double> acc(N, 0.0);
        for (int k = 0; k < K; ++k) {
            const float a = __half2float(A_h[static_cast<size_t>(m) * K + k]);
            if (a != 0.0f)
                for (int n = 0; n < N; ++n)
                    acc[n] += static_cast<double>(a) * Bf[static_cast<size_t>(n) * K + k];
        }
        for (int n = 0; n < N; ++n)
            want[static_cast<size_t>(n) * M + m] = static_cast<float>(acc[n]);
    });
    double total_error = 0.0, sumsq = 0.0;
    for (size_t i = 0; i < want.size(); ++i) {
        total_error += fabs(want[i] - __half2float(C_h[i]));
        sumsq += static_cast<double>(want[i]) * want[i];
    }
    const double floor_v = 0.05 * sqrt(sumsq / want.size());
    double       max_rel = 0.0;
    for (size_t i = 0; i < want.size(); ++i) {
        const double denom = fabs(want[i]) > floor_v ? fabs(want[i]) : floor_v;
        const double rel   = fabs(want[i] - __half2float(C_h[i])) / (denom > 0 ? denom : 1.0);
        max_rel            = rel > max_rel ? rel : max_rel;
    }
    const double tflops = 2.0 * M * N * K / (ms * 1e-3) / 1e12;
    const double bytes  = 4.0 * nnz + 4.0 * num_offsets + 2.0 * K * N + 2.0 * M * N;
    printf("%-10s \t -> \t\t Time/ms: %5.3f \t Performance/TFLOPs: %4.2f \t TotalError: %.2lf\n", "FlashLLM_B200", ms, tflops,
           total_error);

    float ref_ms = -1.f;
    if (ref_path) {
        void* h = dlopen(ref_path, RTLD_NOW | RTLD_LOCAL);
        SpmmFn ref = h ? reinterpret_cast<SpmmFn>(dlsym(h, "_Z15SpMM_SplitK_APIP11CUstream_stPK6__halfPK5uint4PKiS3_PS1_iiiS9_i")) : nullptr;
        if (!ref)
            printf("reference library %s could not be loaded: %s\n", ref_path, dlerror());
        else if (M % 256 != 0)
            printf("reference kernel needs M %% 256 == 0; skipped\n");
        else {
            ref_ms = time_spmm(ref, reinterpret_cast<uint4*>(nz_d), offs_d, B_d, C_d, M, N, K, ws_d, split_k, 20, 200);
            printf("%-10s \t -> \t\t Time/ms: %5.3f \t Performance/TFLOPs: %4.2f\n", "FlashLLM_ref", ref_ms,
                   2.0 * M * N * K / (ref_ms * 1e-3) / 1e12);
        }
    }
    printf("{\"M\": %d, \"K\": %d, \"N\": %d, \"sparsity\": %d, \"split_k\": %d, \"ms\": %.5f, \"tflops_eff\": %.2f, \"gbs\": %.1f, "
           "\"frac_of_8000\": %.3f, \"max_rel_err\": %.3e, \"total_error\": %.3f, \"device_encode_ms\": %.3f, "
           "\"encoders_bit_identical\": %s, \"status\": %u, \"reference_ms\": %.5f}\n",
           M, K, N, sparsity_pct, split_k, ms, tflops, bytes / (ms * 1e-3) / 1e9, bytes / (ms * 1e-3) / 1e9 / 8000.0, max_rel,
           total_error, encode_ms, encoders_agree ? "true" : "false", status, ref_ms);
    free(nz_h);
    free(offs_h);
    return (encoders_agree && status == 0 && max_rel <= 1e-2) ? 0 : 2;
}
