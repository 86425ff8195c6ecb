/*
 * TEST INFRASTRUCTURE — CPU oracle for the Flash-LLM tiled-CSL SpMM path.
 *
 * Plain-C restatement of the reference algorithm, used only as a checker by the test-suite,
 * the smoke test and the benchmark's CPU-baseline leg.  Nothing in the shipped library calls
 * into this file.
 *
 * Parity status: PINNED.  The reference ships no golden vectors for this path; the pin is the
 * reference's own host encoder, compiled unmodified from its sources (see the Makefile beside
 * this file) and compared bit-for-bit with these functions by tests/test_oracle_pin.py, plus
 * fixtures generated from that same build under tests/golden/.
 *
 * Reference files restated here (paths inside the Flash-LLM project):
 *   csrc/SpMM_API.cu:163-360   InitSparseMatrixA_API            -> oracle_encode_reorder
 *   csrc/SpMM_API.cu:363-489   InitSparseMatrixA_API_NoReorder  -> oracle_encode_noreorder
 *   csrc/SpMM_API.cu:132-156   BankID_Minimum / BankID_Maximum  -> bank_min / bank_max
 *   csrc/SpMM_Kernel.cuh:138-177 (word -> smem cell)            -> oracle_decode
 *   csrc/SpMM_Kernel.cuh:191-205,374-385 + csrc/Reduction_Kernel.cuh:24-45
 *                                                               -> oracle_spmm_splitk
 *   kernel_benchmark/spmm_test_utils.h:120-126 ComputeTotalError -> oracle_total_error
 * The dense fp32 GEMM (oracle_gemm_f32) has no counterpart in the reference, whose own check
 * is a cuBLAS GEMM (kernel_benchmark/spmm_test.cu:115-163); it computes the same product
 * C[n][m] = sum_k A[m][k] * B[n][k] on the host.
 */
#include <math.h>
#include <stdint.h>
#include <stdlib.h>
#include <string.h>

#define TILE_M 128
#define TILE_K 64
#define VEC 4

/* ---------------------------------------------------------------- fp16 <-> fp32 */

float oracle_half_to_float(uint16_t h)
{
    uint32_t sign = (uint32_t)(h & 0x8000u) << 16;
    uint32_t exp  = (h >> 10) & 0x1fu;
    uint32_t man  = h & 0x3ffu;
    uint32_t bits;
    if (exp == 0) {
        if (man == 0) {
            bits = sign;
        } else { /* subnormal: normalise */
            int e = -1;
            do {
                e++;
                man <<= 1;
            } while ((man & 0x400u) == 0);
            man &= 0x3ffu;
            bits = sign | ((uint32_t)(127 - 15 - e) << 23) | (man << 13);
        }
    } else if (exp == 31) {
        bits = sign | 0x7f800000u | (man << 13);
    } else {
        bits = sign | ((exp + 127 - 15) << 23) | (man << 13);
    }
    float f;
    memcpy(&f, &bits, 4);
    return f;
}

/* round-to-nearest-even, the behaviour of __float2half_rn */
uint16_t oracle_float_to_half(float f)
{
    uint32_t x;
    memcpy(&x, &f, 4);
    uint32_t sign = (x >> 16) & 0x8000u;
    uint32_t abs  = x & 0x7fffffffu;
    if (abs > 0x7f800000u) return (uint16_t)(sign | 0x7fffu);          /* NaN */
    if (abs >= 0x47800000u) return (uint16_t)(sign | 0x7c00u);         /* >= 65536 -> inf (incl. inf) */
    if (abs >= 0x477ff000u) return (uint16_t)(sign | 0x7c00u);         /* rounds up to inf */
    if (abs < 0x33000000u) return (uint16_t)sign;                      /* < 2^-25 -> 0 */
    if (abs < 0x38800000u) {                                           /* subnormal half */
        int      e     = (int)(abs >> 23);                             /* biased fp32 exponent */
        uint32_t man   = (abs & 0x7fffffu) | 0x800000u;
        int      rs    = 126 - e;                                      /* value = man * 2^(e-150); unit = 2^-24 */
        uint32_t q     = man >> rs;
        uint32_t rem   = man & ((1u << rs) - 1u);
        uint32_t half  = 1u << (rs - 1);
        if (rem > half || (rem == half && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
    {
        uint32_t e   = (abs >> 23) - 112;                              /* half biased exponent */
        uint32_t man = abs & 0x7fffffu;
        uint32_t q   = (e << 10) | (man >> 13);
        uint32_t rem = man & 0x1fffu;
        if (rem > 0x1000u || (rem == 0x1000u && (q & 1u))) q++;
        return (uint16_t)(sign | q);
    }
}

/* The reference's zero test: fabs(__half2float(v)) > 0.0f  (SpMM_API.cu:184,210,257).
 * True for every finite non-zero value and for infinities; false for +-0 and for NaN. */
static int is_nonzero(uint16_t h)
{
    return fabsf(oracle_half_to_float(h)) > 0.0f;
}

/* ---------------------------------------------------------------- bank bookkeeping */

typedef struct {
    uint32_t items[32][TILE_M * TILE_K / 32 + VEC]; /* a bank has 256 cells; <=3 padding words on top */
    int      count[32];
} Banks;

/* SpMM_API.cu:132-143 — first index among the smallest buckets */
static int bank_min(const Banks* b)
{
    int id = 0, best = b->count[0];
    for (int i = 1; i < 32; i++)
        if (b->count[i] < best) {
            id   = i;
            best = b->count[i];
        }
    return id;
}

/* SpMM_API.cu:145-156 — first index among the largest buckets */
static int bank_max(const Banks* b)
{
    int id = 0, best = b->count[0];
    for (int i = 1; i < 32; i++)
        if (b->count[i] > best) {
            id   = i;
            best = b->count[i];
        }
    return id;
}

static uint32_t pack_word(uint16_t value, int loc)
{
    return (uint32_t)value | ((uint32_t)(uint16_t)(int16_t)loc << 16);
}

static int count_tile_nnz(const uint16_t* tile, int K)
{
    int n = 0;
    for (int m = 0; m < TILE_M; m++)
        for (int k = 0; k < TILE_K; k++)
            if (is_nonzero(tile[(size_t)m * K + k])) n++;
    return n;
}

/* ---------------------------------------------------------------- encoder, reordered (SpMM_API.cu:163-360) */

int oracle_encode_reorder(const uint16_t* A, int M, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    if (M % TILE_M != 0 || K % TILE_K != 0) return -1;
    const int rows = M / TILE_M, cols = K / TILE_K;
    const int T = rows * cols;
    int*      pad_of = (int*)malloc((size_t)(T > 0 ? T : 1) * sizeof(int));
    long long padded = 0;
    /* pass 2 of the reference (200-216): per-tile count and padding to a multiple of 4 */
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < cols; j++) {
            int nnz = count_tile_nnz(A + (size_t)i * TILE_M * K + (size_t)j * TILE_K, K);
            int pad = (VEC - nnz % VEC) % VEC;
            pad_of[i * cols + j] = pad;
            padded += nnz + pad;
        }
    uint32_t* out  = (uint32_t*)malloc((size_t)(padded > 0 ? padded : 1) * sizeof(uint32_t));
    int*      offs = (int*)malloc((size_t)(T + 2) * sizeof(int));
    Banks*    bk   = (Banks*)malloc(sizeof(Banks));
    /* the two lane-queue sets of the reference (MainPart / TailPart, 292-293) */
    uint32_t(*mainq)[TILE_M * TILE_K / 32 + VEC] = malloc(sizeof(uint32_t[32][TILE_M * TILE_K / 32 + VEC]));
    uint32_t(*tailq)[VEC]                        = malloc(sizeof(uint32_t[32][VEC]));
    int       main_n[32], tail_n[32];
    long long total = 0;
    uint32_t* dst   = out;
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < cols; j++) {
            const uint16_t* tile = A + (size_t)i * TILE_M * K + (size_t)j * TILE_K;
            int             zero_pos[32];
            int             tile_n = 0;
            for (int b = 0; b < 32; b++) {
                bk->count[b] = 0;
                zero_pos[b]  = -1;
                main_n[b] = tail_n[b] = 0;
            }
            /* bucket by destination bank, row-major scan (248-271) */
            for (int m = 0; m < TILE_M; m++)
                for (int n = 0; n < TILE_K; n++) {
                    uint16_t v    = tile[(size_t)m * K + n];
                    int      colp = n ^ ((m % 8) << 3);
                    int      bank = (colp / 2) % 32;
                    int      loc  = m * TILE_K + colp;
                    if (is_nonzero(v)) {
                        bk->items[bank][bk->count[bank]++] = pack_word(v, loc);
                        tile_n++;
                    } else if (zero_pos[bank] == -1) {
                        zero_pos[bank] = loc;
                    }
                }
            /* padding words: +0.0 aimed at the first zero cell of the emptiest bank (274-287) */
            for (int p = 0; p < pad_of[i * cols + j]; p++) {
                int b = bank_min(bk);
                bk->items[b][bk->count[b]++] = pack_word(0, zero_pos[b]);
                tile_n++;
            }
            const int vectors = tile_n / VEC;
            const int repeat  = vectors / 32;
            const int remain  = vectors % 32;
            /* tail first, then main: always pop the newest item of the fullest bank (299-320) */
            for (int v = 0; v < VEC; v++)
                for (int b = 0; b < remain; b++) {
                    int src = bank_max(bk);
                    tailq[b][tail_n[b]++] = bk->items[src][--bk->count[src]];
                }
            for (int r = 0; r < repeat; r++)
                for (int v = 0; v < VEC; v++)
                    for (int b = 0; b < 32; b++) {
                        int src = bank_max(bk);
                        mainq[b][main_n[b]++] = bk->items[src][--bk->count[src]];
                    }
            /* emit: lane queues are drained newest-first (323-346) */
            for (int r = 0; r < repeat; r++)
                for (int v = 0; v < VEC; v++)
                    for (int b = 0; b < 32; b++) dst[r * VEC * 32 + b * VEC + v] = mainq[b][--main_n[b]];
            dst += (size_t)repeat * VEC * 32;
            for (int v = 0; v < VEC; v++)
                for (int b = 0; b < remain; b++) dst[b * VEC + v] = tailq[b][--tail_n[b]];
            dst += (size_t)VEC * remain;
            total += tile_n;
            offs[i * cols + j + 1] = (int)(total / VEC);
        }
    offs[0]     = 0;
    offs[T + 1] = (int)(total / VEC);
    free(pad_of);
    free(bk);
    free(mainq);
    free(tailq);
    *Compressed_A = out;
    *TileOffsets  = offs;
    return T + 2;
}

/* ---------------------------------------------------------------- encoder, scan order (SpMM_API.cu:363-489) */

int oracle_encode_noreorder(const uint16_t* A, int M, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    if (M % TILE_M != 0 || K % TILE_K != 0) return -1;
    const int rows = M / TILE_M, cols = K / TILE_K;
    const int T = rows * cols;
    long long padded = 0;
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < cols; j++) {
            int nnz = count_tile_nnz(A + (size_t)i * TILE_M * K + (size_t)j * TILE_K, K);
            padded += nnz + (VEC - nnz % VEC) % VEC;
        }
    uint32_t* out  = (uint32_t*)malloc((size_t)(padded > 0 ? padded : 1) * sizeof(uint32_t));
    int*      offs = (int*)malloc((size_t)(T + 2) * sizeof(int));
    long long total = 0;
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < cols; j++) {
            const uint16_t* tile = A + (size_t)i * TILE_M * K + (size_t)j * TILE_K;
            int             nnz  = count_tile_nnz(tile, K);
            int             pads = (VEC - nnz % VEC) % VEC;
            for (int m = 0; m < TILE_M; m++)
                for (int n = 0; n < TILE_K; n++) {
                    uint16_t v   = tile[(size_t)m * K + n];
                    int      loc = m * TILE_K + (n ^ ((m % 8) << 3));
                    if (is_nonzero(v)) {
                        out[total++] = pack_word(v, loc);
                    } else if (pads > 0) { /* the first cells that test as zero become the padding, bits kept (456-472) */
                        pads--;
                        out[total++] = pack_word(v, loc);
                    }
                }
            offs[i * cols + j + 1] = (int)(total / VEC);
        }
    offs[0]     = 0;
    offs[T + 1] = (int)(total / VEC);
    *Compressed_A = out;
    *TileOffsets  = offs;
    return T + 2;
}

void oracle_free(void* p)
{
    free(p);
}

/* ---------------------------------------------------------------- decoder (consumer side, SpMM_Kernel.cuh:138-177) */

/* Rebuilds the dense row-major fp16 matrix: every cell starts at +0.0, then smem[loc] = value per word. */
void oracle_decode(const uint32_t* Compressed_A, const int* TileOffsets, int M, int K, uint16_t* A_out)
{
    const int rows = M / TILE_M, cols = K / TILE_K;
    memset(A_out, 0, (size_t)M * K * sizeof(uint16_t));
    for (int i = 0; i < rows; i++)
        for (int j = 0; j < cols; j++) {
            int       t     = i * cols + j;
            long long begin = (long long)TileOffsets[t] * VEC, end = (long long)TileOffsets[t + 1] * VEC;
            for (long long w = begin; w < end; w++) {
                uint32_t word = Compressed_A[w];
                int      loc  = (int)(word >> 16);
                int      r    = loc >> 6;
                int      c    = (loc & 63) ^ ((r & 7) << 3);
                A_out[((size_t)i * TILE_M + r) * K + (size_t)j * TILE_K + c] = (uint16_t)(word & 0xffffu);
            }
        }
}

/* ---------------------------------------------------------------- host dense GEMM */

/* Number of host threads the OpenMP loops below use.  A launcher may have pinned OMP_NUM_THREADS to 1 in the
 * environment (torch.distributed.run does); callers that time the host path on all cores set it back here. */
#ifdef _OPENMP
#include <omp.h>
#endif
void oracle_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0)
        omp_set_num_threads(n);
#else
    (void)n;
#endif
}


/* C[n][m] = sum_k float(A[m][k]) * float(B[n][k]); rows [m_begin, m_end) only, double accumulation,
 * result stored as float.  A row-major [M][K], B row-major [N][K], C row-major [N][M]. */
void oracle_gemm_f32(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K, int m_begin, int m_end)
{
    float* Bf = (float*)malloc((size_t)N * K * sizeof(float));
    for (size_t i = 0; i < (size_t)N * K; i++) Bf[i] = oracle_half_to_float(B[i]);
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = m_begin; m < m_end; m++) {
            for (int k = 0; k < K; k++) row[k] = oracle_half_to_float(A[(size_t)m * K + k]);
            for (int n = 0; n < N; n++) {
                const float* b   = Bf + (size_t)n * K;
                double       acc = 0.0;
                for (int k = 0; k < K; k++) acc += (double)row[k] * (double)b[k];
                C[(size_t)n * M + m] = (float)acc;
            }
        }
        free(row);
    }
    free(Bf);
}

/* The same product in single precision with a dense inner loop: the timed CPU baseline. */
void oracle_gemm_f32_timed(const uint16_t* A, const uint16_t* B, float* C, int M, int N, int K, int m_begin, int m_end)
{
    float* Bf = (float*)malloc((size_t)N * K * sizeof(float));
    for (size_t i = 0; i < (size_t)N * K; i++) Bf[i] = oracle_half_to_float(B[i]);
#pragma omp parallel
    {
        float* row = (float*)malloc((size_t)K * sizeof(float));
#pragma omp for schedule(static)
        for (int m = m_begin; m < m_end; m++) {
            for (int k = 0; k < K; k++) row[k] = oracle_half_to_float(A[(size_t)m * K + k]);
            for (int n = 0; n < N; n++) {
                const float* b   = Bf + (size_t)n * K;
                float        acc = 0.0f;
#pragma omp simd reduction(+ : acc)
                for (int k = 0; k < K; k++) acc += row[k] * b[k];
                C[(size_t)n * M + m] = acc;
            }
        }
        free(row);
    }
    free(Bf);
}

/* ---------------------------------------------------------------- SpMM with the reference's split-K semantics */

/* Walks the compressed stream the way the kernel does: K batch b of Split_K covers k-tiles
 * [b*avg, b*avg + iters) with avg = ceil((K/64)/Split_K) and the last batch shortened by the
 * round-up (SpMM_Kernel.cuh:191-205).  Each batch accumulates in fp32 and, when Split_K > 1,
 * is rounded to fp16 (374-385) before the fp32 sum over batches and the final fp16 rounding
 * (Reduction_Kernel.cuh:24-45).  C is row-major [N][M] fp16.  Returns 0, or -1 if a batch
 * would be empty or start past the matrix (configurations the reference kernel cannot run). */
int oracle_spmm_splitk(const uint32_t* Compressed_A, const int* TileOffsets, const uint16_t* B, uint16_t* C,
                       int M, int N, int K, int Split_K)
{
    const int cols = K / TILE_K, rows = M / TILE_M;
    const int avg  = (cols - 1) / Split_K + 1;
    const int padk = avg * Split_K - cols;
    if (avg - padk <= 0) return -1;
    float* Bf = (float*)malloc((size_t)N * K * sizeof(float));
    for (size_t i = 0; i < (size_t)N * K; i++) Bf[i] = oracle_half_to_float(B[i]);
#pragma omp parallel
    {
        float* acc   = (float*)malloc((size_t)TILE_M * N * sizeof(float));
        float* total = (float*)malloc((size_t)TILE_M * N * sizeof(float));
#pragma omp for schedule(dynamic)
        for (int i = 0; i < rows; i++) {
            for (int e = 0; e < TILE_M * N; e++) total[e] = 0.0f;
            for (int b = 0; b < Split_K; b++) {
                int iters = (b == Split_K - 1) ? avg - padk : avg;
                for (int e = 0; e < TILE_M * N; e++) acc[e] = 0.0f;
                for (int kk = 0; kk < iters; kk++) {
                    int       j     = b * avg + kk;
                    int       t     = i * cols + j;
                    long long begin = (long long)TileOffsets[t] * VEC, end = (long long)TileOffsets[t + 1] * VEC;
                    for (long long w = begin; w < end; w++) {
                        uint32_t word = Compressed_A[w];
                        int      loc  = (int)(word >> 16);
                        int      r    = loc >> 6;
                        int      c    = (loc & 63) ^ ((r & 7) << 3);
                        float    v    = oracle_half_to_float((uint16_t)(word & 0xffffu));
                        size_t   kcol = (size_t)j * TILE_K + c;
                        for (int n = 0; n < N; n++) acc[n * TILE_M + r] += v * Bf[(size_t)n * K + kcol];
                    }
                }
                if (Split_K == 1) {
                    for (int e = 0; e < TILE_M * N; e++) total[e] = acc[e];
                } else {
                    for (int e = 0; e < TILE_M * N; e++)
                        total[e] += oracle_half_to_float(oracle_float_to_half(acc[e]));
                }
            }
            for (int n = 0; n < N; n++)
                for (int r = 0; r < TILE_M; r++)
                    C[(size_t)n * M + (size_t)i * TILE_M + r] = oracle_float_to_half(total[n * TILE_M + r]);
        }
        free(acc);
        free(total);
    }
    free(Bf);
    return 0;
}

/* kernel_benchmark/spmm_test_utils.h:120-126 */
double oracle_total_error(const uint16_t* ref, const uint16_t* other, long long count)
{
    double e = 0.0;
    for (long long i = 0; i < count; i++)
        e += fabs((double)oracle_half_to_float(ref[i]) - (double)oracle_half_to_float(other[i]));
    return e;
}
