// Host tiled-CSL encoder (see tiled_csl_host.cpp).
#pragma once
#include <cstdint>

namespace flashllm {

// Dense row-major fp16 bit patterns -> tiled-CSL.  Both outputs are malloc'ed.  Returns (M/128)*(K/64) + 2, or
// -1 for bad arguments (M % 128, K % 64, null pointers), -2 when out of memory, -3 when the matrix holds more
// 16-byte vectors than the format's int offsets can count.
int encode_tiled_csl_host(const uint16_t* A, int M, int K, bool reorder, uint32_t** Compressed_A, int** TileOffsets);

// Counts kernel launches for FlashLLM_LaunchCount.
void count_launch();

// Device address of the current device's status word (set up on first use); returns a cudaError_t value.
int device_status_pointer(unsigned int** status);

}  // namespace flashllm
