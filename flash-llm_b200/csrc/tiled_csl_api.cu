// Encoder entry points of libSpMM_API.so: the reference-named host encoders and file converter
// (reference csrc/SpMM_API.cu:163-555) and their C-linkage aliases.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
#include <string>
#include <vector>

#include "../../include/SpMM_API.cuh"
#include "tiled_csl_device.cuh"
#include "tiled_csl_host.h"
#include "tiling.h"

using namespace flashllm;

// The reference reports allocation failures with a message and exit(-1) (csrc/SpMM_API.cu:196-199,227-230) and
// asserts on the tile divisibility (:232); the reference-named entry points keep that behaviour.
static int encode_or_exit(const half* A_h, int M, int K, bool reorder, uint32_t** Compressed_A, int** TileOffsets)
{
    const int n = encode_tiled_csl_host(reinterpret_cast<const uint16_t*>(A_h), M, K, reorder, Compressed_A, TileOffsets);
    if (n == -1) {
        printf("InitSparseMatrixA: M (%d) must be a positive multiple of 128 and K (%d) of 64.\n", M, K);
        exit(-1);
    }
    if (n == -2) {
        printf("InitSparseMatrixA: Error in malloc memory from host memory!\n");
        exit(-1);
    }
    if (n == -3) {
        printf("InitSparseMatrixA: matrix too large for 32-bit TileOffsets.\n");
        exit(-1);
    }
    return n;
}

__host__ int InitSparseMatrixA_API(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_or_exit(A_h, M, K, true, Compressed_A, TileOffsets);
}

__host__ int
InitSparseMatrixA_API_NoReorder(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_or_exit(A_h, M, K, false, Compressed_A, TileOffsets);
}

extern "C" {

int FlashLLM_InitSparseMatrixA(const void* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets)
{
    (void)N;
    return encode_tiled_csl_host(static_cast<const uint16_t*>(A_h), M, K, true, Compressed_A, TileOffsets);
}

int FlashLLM_InitSparseMatrixA_NoReorder(const void* A_h, int M, int N, int K, uint32_t** Compressed_A,
                                         int** TileOffsets)
{
    (void)N;
    return encode_tiled_csl_host(static_cast<const uint16_t*>(A_h), M, K, false, Compressed_A, TileOffsets);
}

int FlashLLM_EncodeOnDevice_TileOffsets(void* stream, const void* A_d, int M, int K, int* TileOffsets_d)
{
    if (A_d == nullptr || TileOffsets_d == nullptr || M <= 0 || K <= 0 || M % kTileM != 0 || K % kTileK != 0
        || (reinterpret_cast<uintptr_t>(A_d) & 3u) != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    unsigned int* status = nullptr;
    if (int rc = device_status_pointer(&status))
        return rc;
    const int    k_tiles = K / kTileK, tiles = (M / kTileM) * k_tiles;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    count_launch();
    csl_count_kernel<<<(tiles + kEncodeWarps - 1) / kEncodeWarps, kEncodeWarps * 32, 0, s>>>(
        static_cast<const uint16_t*>(A_d), K, tiles, k_tiles, TileOffsets_d);
    count_launch();
    csl_scan_kernel<<<1, 1024, 0, s>>>(TileOffsets_d, tiles, status);
    return static_cast<int>(cudaGetLastError());
}

int FlashLLM_EncodeOnDevice_Pack(void* stream, const void* A_d, int M, int K, const int* TileOffsets_d,
                                 uint32_t* Compressed_A_d, int reorder)
{
    if (A_d == nullptr || TileOffsets_d == nullptr || Compressed_A_d == nullptr || M <= 0 || K <= 0 || M % kTileM != 0
        || K % kTileK != 0 || (reinterpret_cast<uintptr_t>(A_d) & 3u) != 0)
        return static_cast<int>(cudaErrorInvalidValue);
    unsigned int* status = nullptr;
    if (int rc = device_status_pointer(&status))
        return rc;
    const int    k_tiles = K / kTileK, tiles = (M / kTileM) * k_tiles;
    const int    blocks  = (tiles + kEncodeWarps - 1) / kEncodeWarps;
    cudaStream_t s       = static_cast<cudaStream_t>(stream);
    count_launch();
    if (reorder)
        csl_pack_reorder_kernel<<<blocks, kEncodeWarps * 32, 0, s>>>(static_cast<const uint16_t*>(A_d), K, tiles, k_tiles,
                                                                      TileOffsets_d, Compressed_A_d, status);
    else
        csl_pack_scan_kernel<<<blocks, kEncodeWarps * 32, 0, s>>>(static_cast<const uint16_t*>(A_d), K, tiles, k_tiles,
                                                                   TileOffsets_d, Compressed_A_d, status);
    return static_cast<int>(cudaGetLastError());
}

void FlashLLM_Free(void* p)
{
    free(p);
}

void GenSparseMatrixBinFile(char* DenseMatrixFileName,
                            int   M,
                            int   K,
                            char* NZWeightsFileName,
                            char* TileOffsetsFileName,
                            char* OutputSizesFileName)
{
    const size_t      elems = static_cast<size_t>(M) * static_cast<size_t>(K);
    std::vector<half> dense(elems);
    std::ifstream     in(DenseMatrixFileName, std::ios::in | std::ios::binary);
    if (!in.is_open()) {
        printf("file %s cannot be opened, loadDataArrayFromBin fails. \n", DenseMatrixFileName);
        exit(-1);
    }
    const size_t want = sizeof(half) * elems;
    in.read(reinterpret_cast<char*>(dense.data()), static_cast<std::streamsize>(want));
    const size_t got = static_cast<size_t>(in.gcount());
    if (got != want) {
        printf("file %s only has %ld, but request %ld, loading DenseMatrix fails! \n", DenseMatrixFileName,
               static_cast<long>(got), static_cast<long>(want));
        exit(-1);
    }
    in.close();
    uint32_t* words   = nullptr;
    int*      offsets = nullptr;
    const int num_offsets = InitSparseMatrixA_API(dense.data(), M, 0, K, &words, &offsets);
    const int nnz         = offsets[num_offsets - 1] * kVectorWords;
    std::ofstream sizes(OutputSizesFileName, std::ios::out | std::ios::binary);
    std::ofstream weights(NZWeightsFileName, std::ios::out | std::ios::binary);
    std::ofstream offs(TileOffsetsFileName, std::ios::out | std::ios::binary);
    if (!sizes.is_open() || !weights.is_open() || !offs.is_open()) {
        printf("GenSparseMatrixBinFile() ERROR: file %s, %s, or %s cannot be opened or creaetd. \n", OutputSizesFileName,
               NZWeightsFileName, TileOffsetsFileName);
        exit(-1);
    }
    sizes.write(reinterpret_cast<const char*>(&nnz), sizeof(int));
    sizes.write(reinterpret_cast<const char*>(&num_offsets), sizeof(int));
    weights.write(reinterpret_cast<const char*>(words), static_cast<std::streamsize>(sizeof(uint32_t)) * nnz);
    offs.write(reinterpret_cast<const char*>(offsets), static_cast<std::streamsize>(sizeof(int)) * num_offsets);
    free(words);
    free(offsets);
}

// ------------------------------------------------------------------------------------------------------------
// On-disk format: the three files GenSparseMatrixBinFile writes per matrix and the three per-rank lists the
// reference's converter writes per model directory (end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:
// 52-59,188-195), as FasterTransformer loads them (third_party/ft.patch:1863-1965, loadDataArrayFromBin :3743-3790).
// Result codes: 0 ok, -1 a file cannot be opened or created, -2 a file is shorter than asked for, -3 the contents
// are not a well-formed tiled-CSL matrix, -4 bad arguments, positive = cudaError_t.
// ------------------------------------------------------------------------------------------------------------

static int read_exact(const char* name, void* dst, size_t bytes)
{
    std::ifstream in(name, std::ios::in | std::ios::binary);
    if (!in.is_open())
        return -1;
    in.read(static_cast<char*>(dst), static_cast<std::streamsize>(bytes));
    return static_cast<size_t>(in.gcount()) == bytes ? 0 : -2;
}

static int write_exact(const char* name, const void* src, size_t bytes)
{
    std::ofstream out(name, std::ios::out | std::ios::binary);
    if (!out.is_open())
        return -1;
    out.write(static_cast<const char*>(src), static_cast<std::streamsize>(bytes));
    return out.good() ? 0 : -1;
}

// TileOffsets as the kernels expect them: start at 0, never run backwards, at most 2048 vectors per tile, an empty
// sentinel tile at the end, and a word count that agrees with OutputSizes.
static bool offsets_well_formed(const int* offs, int num_offsets, int nnz)
{
    if (num_offsets < kOffsetsExtra + 1 || offs[0] != 0)
        return false;
    for (int i = 0; i + 1 < num_offsets; ++i)
        if (offs[i + 1] < offs[i] || offs[i + 1] - offs[i] > kMaxTileVectors)
            return false;
    return offs[num_offsets - 1] == offs[num_offsets - 2]
           && static_cast<long long>(offs[num_offsets - 1]) * kVectorWords == static_cast<long long>(nnz);
}

int FlashLLM_ReadOutputSizes(const char* OutputSizesFileName, int* NNZ, int* NumOffsets)
{
    if (OutputSizesFileName == nullptr || NNZ == nullptr || NumOffsets == nullptr)
        return -4;
    int pair[2] = {0, 0};
    if (int rc = read_exact(OutputSizesFileName, pair, sizeof(pair)))
        return rc;
    if (pair[0] < 0 || pair[1] < kOffsetsExtra + 1 || pair[0] % kVectorWords != 0)
        return -3;
    *NNZ        = pair[0];
    *NumOffsets = pair[1];
    return 0;
}

int FlashLLM_ReadSparseMatrixBinFiles(const char* NZWeightsFileName, const char* TileOffsetsFileName, int NNZ,
                                      int NumOffsets, uint32_t* Compressed_A_h, int* TileOffsets_h)
{
    if (NZWeightsFileName == nullptr || TileOffsetsFileName == nullptr || NNZ < 0 || NumOffsets < kOffsetsExtra + 1
        || TileOffsets_h == nullptr || (NNZ > 0 && Compressed_A_h == nullptr))
        return -4;
    if (int rc = read_exact(TileOffsetsFileName, TileOffsets_h, sizeof(int) * static_cast<size_t>(NumOffsets)))
        return rc;
    if (!offsets_well_formed(TileOffsets_h, NumOffsets, NNZ))
        return -3;
    if (NNZ > 0)
        if (int rc = read_exact(NZWeightsFileName, Compressed_A_h, sizeof(uint32_t) * static_cast<size_t>(NNZ)))
            return rc;
    return 0;
}

int FlashLLM_LoadSparseMatrixBinFiles(const char* NZWeightsFileName, const char* TileOffsetsFileName, int NNZ,
                                      int NumOffsets, void* Compressed_A_d, int* TileOffsets_d)
{
    if (TileOffsets_d == nullptr || (NNZ > 0 && Compressed_A_d == nullptr) || NNZ < 0 || NumOffsets < kOffsetsExtra + 1)
        return -4;
    std::vector<uint32_t> words(static_cast<size_t>(NNZ));
    std::vector<int>      offs(static_cast<size_t>(NumOffsets));
    if (int rc = FlashLLM_ReadSparseMatrixBinFiles(NZWeightsFileName, TileOffsetsFileName, NNZ, NumOffsets, words.data(),
                                                   offs.data()))
        return rc;
    cudaError_t e = cudaMemcpy(TileOffsets_d, offs.data(), sizeof(int) * offs.size(), cudaMemcpyHostToDevice);
    if (e == cudaSuccess && NNZ > 0)
        e = cudaMemcpy(Compressed_A_d, words.data(), sizeof(uint32_t) * words.size(), cudaMemcpyHostToDevice);
    return static_cast<int>(e);
}

static std::string rank_list_name(const char* dir, const char* what, int rank)
{
    return std::string(dir) + "/" + what + "." + std::to_string(rank) + ".bin";
}

int FlashLLM_WriteRankLists(const char* ModelDir, int Rank, int Entries, const int* NNZ_List, const int* NumOffsets_List,
                            const int* SplitK_List)
{
    if (ModelDir == nullptr || Rank < 0 || Entries < 0 || NNZ_List == nullptr || NumOffsets_List == nullptr
        || SplitK_List == nullptr)
        return -4;
    const size_t bytes = sizeof(int) * static_cast<size_t>(Entries);
    if (int rc = write_exact(rank_list_name(ModelDir, "NNZ_List", Rank).c_str(), NNZ_List, bytes))
        return rc;
    if (int rc = write_exact(rank_list_name(ModelDir, "NumOffsets_List", Rank).c_str(), NumOffsets_List, bytes))
        return rc;
    return write_exact(rank_list_name(ModelDir, "SplitK_List", Rank).c_str(), SplitK_List, bytes);
}

int FlashLLM_ReadRankLists(const char* ModelDir, int Rank, int Entries, int* NNZ_List, int* NumOffsets_List,
                           int* SplitK_List)
{
    if (ModelDir == nullptr || Rank < 0 || Entries < 0 || NNZ_List == nullptr || NumOffsets_List == nullptr
        || SplitK_List == nullptr)
        return -4;
    const size_t bytes = sizeof(int) * static_cast<size_t>(Entries);
    if (int rc = read_exact(rank_list_name(ModelDir, "NNZ_List", Rank).c_str(), NNZ_List, bytes))
        return rc;
    if (int rc = read_exact(rank_list_name(ModelDir, "NumOffsets_List", Rank).c_str(), NumOffsets_List, bytes))
        return rc;
    if (int rc = read_exact(rank_list_name(ModelDir, "SplitK_List", Rank).c_str(), SplitK_List, bytes))
        return rc;
    // a matrix left dense is recorded as three zeros; a converted one has all three positive
    for (int i = 0; i < Entries; ++i) {
        const bool dense  = NNZ_List[i] == 0 && NumOffsets_List[i] == 0 && SplitK_List[i] == 0;
        const bool sparse = NNZ_List[i] >= 0 && NNZ_List[i] % kVectorWords == 0 && NumOffsets_List[i] >= kOffsetsExtra + 1
                            && SplitK_List[i] >= 1;
        if (!dense && !sparse)
            return -3;
    }
    return 0;
}

int FlashLLM_GenSparseMatrixBinFile_Device(const char* DenseMatrixFileName, int M, int K, const char* NZWeightsFileName,
                                           const char* TileOffsetsFileName, const char* OutputSizesFileName)
{
    if (DenseMatrixFileName == nullptr || NZWeightsFileName == nullptr || TileOffsetsFileName == nullptr
        || OutputSizesFileName == nullptr || M <= 0 || K <= 0 || M % kTileM != 0 || K % kTileK != 0)
        return -4;
    const size_t          elems = static_cast<size_t>(M) * static_cast<size_t>(K);
    std::vector<uint16_t> dense(elems);
    if (int rc = read_exact(DenseMatrixFileName, dense.data(), sizeof(uint16_t) * elems))
        return rc;
    const int num_offsets = (M / kTileM) * (K / kTileK) + kOffsetsExtra;
    uint16_t* A_d    = nullptr;
    int*      offs_d = nullptr;
    uint32_t* comp_d = nullptr;
    std::vector<int>      offs(static_cast<size_t>(num_offsets));
    std::vector<uint32_t> words;
    int                   nnz = 0;
    cudaError_t           e   = cudaMalloc(&A_d, sizeof(uint16_t) * elems);
    if (e == cudaSuccess)
        e = cudaMalloc(&offs_d, sizeof(int) * offs.size());
    if (e == cudaSuccess)
        e = cudaMemcpy(A_d, dense.data(), sizeof(uint16_t) * elems, cudaMemcpyHostToDevice);
    if (e == cudaSuccess)
        e = static_cast<cudaError_t>(FlashLLM_EncodeOnDevice_TileOffsets(nullptr, A_d, M, K, offs_d));
    if (e == cudaSuccess)
        e = cudaMemcpy(offs.data(), offs_d, sizeof(int) * offs.size(), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess) {
        nnz = offs[num_offsets - 1] * kVectorWords;
        words.resize(static_cast<size_t>(nnz));
        e = cudaMalloc(&comp_d, sizeof(uint32_t) * (words.empty() ? 4 : words.size()));
    }
    if (e == cudaSuccess)
        e = static_cast<cudaError_t>(FlashLLM_EncodeOnDevice_Pack(nullptr, A_d, M, K, offs_d, comp_d, 1));
    if (e == cudaSuccess && nnz > 0)
        e = cudaMemcpy(words.data(), comp_d, sizeof(uint32_t) * words.size(), cudaMemcpyDeviceToHost);
    if (e == cudaSuccess)
        e = cudaDeviceSynchronize();
    cudaFree(A_d);
    cudaFree(offs_d);
    cudaFree(comp_d);
    if (e != cudaSuccess)
        return static_cast<int>(e);
    const int pair[2] = {nnz, num_offsets};
    if (int rc = write_exact(OutputSizesFileName, pair, sizeof(pair)))
        return rc;
    if (int rc = write_exact(NZWeightsFileName, words.data(), sizeof(uint32_t) * words.size()))
        return rc;
    return write_exact(TileOffsetsFileName, offs.data(), sizeof(int) * offs.size());
}

}  // extern "C"
