// Encoder entry points of libSpMM_API.so: the reference-named host encoders and file converter
// (reference csrc/SpMM_API.cu:163-555) and their C-linkage aliases.
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdio>
#include <cstdlib>
#include <fstream>
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

}  // extern "C"
