/*
 * Public interface of libSpMM_API.so — Load-as-Sparse / Compute-as-Dense SpMM for NVIDIA B200 (sm_100a).
 *
 * Drop-in for Flash-LLM's build/SpMM_API.cuh: the first four declarations keep the reference's names,
 * argument order, C++ linkage and meaning, so an object file compiled against the reference header links
 * against this library unchanged.  Every entry point is also exported with C linkage (plain pointers and
 * sizes, `int` carrying a cudaError_t) for FFI callers; those are the symbols a ctypes / cgo / JNI binding
 * would bind.  Matrix layouts are the reference's:
 *     A  row-major [M][K] fp16 (weights; only its tiled-CSL encoding is read by the kernel)
 *     B  row-major [N][K] fp16 ("column-major K x N": tokens x hidden)
 *     C  row-major [N][M] fp16 ("column-major M x N")
 *     C[n][m] = sum_k A[m][k] * B[n][k], fp32 accumulation, one fp16 rounding at the end.
 *
 * Tiled-CSL: A is cut into 128x64 tiles, tile id t = (m/128)*(K/64) + k/64.  Each nonzero is one 32-bit word,
 * low half = fp16 bits, high half = r*64 + (c ^ ((r & 7) << 3)) for the in-tile cell (r, c).  A tile's words
 * are padded with zero-valued words to a multiple of four.  TileOffsets[t] counts 16-byte vectors before tile
 * t; it has T+2 entries and the last two are equal.
 */
#pragma once
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

/* ------------------------------------------------------------------------------------------------------------
 * Reference-compatible C++ entry points
 * ---------------------------------------------------------------------------------------------------------- */

/* Replaces SpMM_SplitK_API (reference build/SpMM_API.cuh:38-48, csrc/SpMM_API.cu:55-130).
 * All pointers are device pointers.  `A` is never read (callers pass nullptr).  Enqueues on `stream` and
 * returns without synchronising.  N must be 8, 16, 32, 64 or a multiple of 128 (otherwise the reference's
 * message is printed and cudaErrorUnknown returned); M % 128 == 0 and K % 64 == 0 (the reference kernel needs
 * M % 256 == 0 for N <= 32; this one does not).  Split_K >= 1 is a hint: K is cut only as far as it takes to fill
 * the GPU, into up to Split_K/2 parts whose fp32 partial matrices are parked in Reduction_Workspace (>= Split_K*M*N
 * halves, 16-byte aligned; may be nullptr when Split_K == 1) and summed by a second kernel that rounds to fp16 once,
 * and/or into parts of a thread-block cluster that are summed in fp32 through distributed shared memory. */
cudaError_t SpMM_SplitK_API(cudaStream_t stream,
                            const half*  A,
                            const uint4* Compressed_A,
                            const int*   TileOffsets,
                            const half*  B,
                            half*        C,
                            const int    M_Global,
                            const int    N_Global,
                            const int    K_Global,
                            half*        Reduction_Workspace,
                            int          Split_K);

/* Replaces InitSparseMatrixA_API (reference build/SpMM_API.cuh:51, csrc/SpMM_API.cu:163-360).
 * Host encoder, dense fp16 -> tiled-CSL with the bank-aware in-tile ordering.  Output is bit-identical to the
 * reference's.  Both outputs are malloc'ed; the caller frees them with free().  `N` is ignored.  Returns the
 * number of TileOffsets entries, (M/128)*(K/64) + 2.  Prints and exits on allocation failure, as the
 * reference does. */
__host__ int InitSparseMatrixA_API(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets);

/* Replaces InitSparseMatrixA_API_NoReorder (reference build/SpMM_API.cuh:53-58, csrc/SpMM_API.cu:363-489):
 * same format, words in row-major scan order. */
__host__ int
InitSparseMatrixA_API_NoReorder(half* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets);

extern "C" {

/* Replaces GenSparseMatrixBinFile (definition at reference csrc/SpMM_API.cu:500-555, called through ctypes with
 * these six arguments by end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:52-59; the reference
 * header's seven-argument prototype does not match its own definition).  Reads M*K fp16 from the dense file and
 * writes {NNZ, NumOffsets} as two int32, NNZ uint32 words, and NumOffsets int32 offsets. */
void GenSparseMatrixBinFile(char* DenseMatrixFileName,
                            int   M,
                            int   K,
                            char* NZWeightsFileName,
                            char* TileOffsetsFileName,
                            char* OutputSizesFileName);

/* ------------------------------------------------------------------------------------------------------------
 * C-ABI aliases (FFI).  `int` results are cudaError_t values unless stated otherwise.
 * ---------------------------------------------------------------------------------------------------------- */

/* C-linkage form of SpMM_SplitK_API (reference csrc/SpMM_API.cu:55). `stream` is a cudaStream_t. */
int FlashLLM_SpMM_SplitK(void*       stream,
                         const void* A,
                         const void* Compressed_A,
                         const int*  TileOffsets,
                         const void* B,
                         void*       C,
                         int         M,
                         int         N,
                         int         K,
                         void*       Reduction_Workspace,
                         int         Split_K);

/* C-linkage forms of the host encoders (reference csrc/SpMM_API.cu:163 and :363); return NumOffsets. */
int FlashLLM_InitSparseMatrixA(const void* A_h, int M, int N, int K, uint32_t** Compressed_A, int** TileOffsets);
int FlashLLM_InitSparseMatrixA_NoReorder(const void* A_h, int M, int N, int K, uint32_t** Compressed_A,
                                         int** TileOffsets);
/* free() for buffers returned by the two encoders above, for callers without access to the C allocator. */
void FlashLLM_Free(void* p);

/* Device encoder, step 1 (device-side counterpart of the counting passes, reference csrc/SpMM_API.cu:200-216):
 * fills TileOffsets_d[0 .. T+1] (T+2 ints) from the dense row-major fp16 device matrix A_d.  Stream-ordered, no
 * scratch memory; bit-identical to the host encoder's TileOffsets. */
int FlashLLM_EncodeOnDevice_TileOffsets(void* stream, const void* A_d, int M, int K, int* TileOffsets_d);

/* Device encoder, step 2 (device-side counterpart of reference csrc/SpMM_API.cu:236-350): writes the packed
 * words, bit-identical to InitSparseMatrixA_API (reorder != 0) or InitSparseMatrixA_API_NoReorder (reorder == 0).
 * Compressed_A_d must hold 4*TileOffsets[T+1] words (read TileOffsets_d[T+1] back after step 1 to size it). */
int FlashLLM_EncodeOnDevice_Pack(void* stream, const void* A_d, int M, int K, const int* TileOffsets_d,
                                 uint32_t* Compressed_A_d, int reorder);

/* ------------------------------------------------------------------------------------------------------------
 * On-disk format (the files of the reference's model converter).  `int` results: 0 ok, -1 a file cannot be opened
 * or created, -2 a file is shorter than asked for, -3 the contents are not a well-formed tiled-CSL matrix,
 * -4 bad arguments, positive = cudaError_t.
 * ---------------------------------------------------------------------------------------------------------- */

/* GenSparseMatrixBinFile with the encoding done on the current CUDA device (reference csrc/SpMM_API.cu:500-555 does
 * it on one CPU thread; the reference's converter spreads matrices over processes instead,
 * end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:147-156).  Same six arguments, byte-identical output
 * files; allocates and frees its device buffers itself and returns a code instead of exiting. */
int FlashLLM_GenSparseMatrixBinFile_Device(const char* DenseMatrixFileName,
                                           int         M,
                                           int         K,
                                           const char* NZWeightsFileName,
                                           const char* TileOffsetsFileName,
                                           const char* OutputSizesFileName);

/* Reads the {NNZ, NumOffsets} pair of an .OutputSizes.bin file (written at reference csrc/SpMM_API.cu:536-541, read
 * back by huggingface_opt_convert_Phase2.py:160-165). */
int FlashLLM_ReadOutputSizes(const char* OutputSizesFileName, int* NNZ, int* NumOffsets);

/* Reads NNZ words of an .NZWeights.bin file and NumOffsets ints of a .TileOffsets.bin file into host buffers of the
 * caller (the host half of FasterTransformer's loadDataArrayFromBin, reference third_party/ft.patch:3743-3790), and
 * checks what that loader does not: offsets start at 0, never run backwards, stay within 2048 vectors per tile, end
 * with the empty sentinel tile and add up to NNZ. */
int FlashLLM_ReadSparseMatrixBinFiles(const char* NZWeightsFileName,
                                      const char* TileOffsetsFileName,
                                      int         NNZ,
                                      int         NumOffsets,
                                      uint32_t*   Compressed_A_h,
                                      int*        TileOffsets_h);

/* The same into device buffers of the caller, ready for SpMM_SplitK_API (reference third_party/ft.patch:1863-1965
 * loads each decoder-layer matrix this way); synchronous copies on the current device. */
int FlashLLM_LoadSparseMatrixBinFiles(const char* NZWeightsFileName,
                                      const char* TileOffsetsFileName,
                                      int         NNZ,
                                      int         NumOffsets,
                                      void*       Compressed_A_d,
                                      int*        TileOffsets_d);

/* The per-rank lists of a converted model directory: NNZ_List.<rank>.bin, NumOffsets_List.<rank>.bin and
 * SplitK_List.<rank>.bin, `Entries` int32 each (4 per decoder layer, in the order QKV, attention output, FFN1, FFN2;
 * a matrix left dense is recorded as 0/0/0).  Written at huggingface_opt_convert_Phase2.py:188-195, read by the
 * patched FasterTransformer (third_party/ft.patch:2357-2359). */
int FlashLLM_WriteRankLists(const char* ModelDir,
                            int         Rank,
                            int         Entries,
                            const int*  NNZ_List,
                            const int*  NumOffsets_List,
                            const int*  SplitK_List);
int FlashLLM_ReadRankLists(const char* ModelDir, int Rank, int Entries, int* NNZ_List, int* NumOffsets_List,
                           int* SplitK_List);

/* SpMM with the output epilogue of the reference's feed-forward call sites fused in (no counterpart in the reference
 * library: FasterTransformer runs add-bias + ReLU as a separate pass over C after the first FFN GEMM,
 * third_party/ft.patch ParallelGpt FFN layer): C[n][m] = act(sum_k A[m][k] * B[n][k] + bias[m]), computed on the fp32
 * sum and rounded to fp16 once.  `bias` is a device pointer to M halves or nullptr; `activation` 0 = none, 1 = ReLU.
 * Other arguments and results as FlashLLM_SpMM_SplitK (without the unused `A`). */
int FlashLLM_SpMM_SplitK_BiasAct(void*       stream,
                                 const void* Compressed_A,
                                 const int*  TileOffsets,
                                 const void* B,
                                 void*       C,
                                 int         M,
                                 int         N,
                                 int         K,
                                 void*       Reduction_Workspace,
                                 int         Split_K,
                                 const void* bias,
                                 int         activation);

/* The same with the residual of the decoder layer added as well (FasterTransformer's add_bias_residual pass after the
 * attention output projection and after the second FFN GEMM, third_party/ft.patch FfnLayer / ParallelGpt call sites):
 * C[n][m] = fp16(act(sum + bias[m]) + residual[n][m]).  `residual` is a device matrix laid out like C that does not
 * overlap it, or nullptr (then identical to FlashLLM_SpMM_SplitK_BiasAct). */
int FlashLLM_SpMM_SplitK_Epilogue(void*       stream,
                                  const void* Compressed_A,
                                  const int*  TileOffsets,
                                  const void* B,
                                  void*       C,
                                  int         M,
                                  int         N,
                                  int         K,
                                  void*       Reduction_Workspace,
                                  int         Split_K,
                                  const void* bias,
                                  int         activation,
                                  const void* residual);

/* ------------------------------------------------------------------------------------------------------------
 * Row-parallel SpMM with the all-reduce fused in (tensor-parallel inference: the attention output projection and
 * the second feed-forward matmul hold a slice of K on every GPU, so every GPU's product is a partial sum).  The
 * reference's caller runs the SpMM and then FasterTransformer's NCCL all-reduce (third_party/ft.patch:2822-2846 and
 * the call sites :1328-1340, :615-633; its custom all-reduce is switched off, :97).  Here the SpMM kernel stores its
 * fp32 partial sums straight into a receive buffer on every GPU of the group (plain peer stores over NVLink) and
 * raises a flag per CTA (per output tile when the GPU's own K range is cut into parts: the parts are parked in the GPU's
 * own buffer and the last CTA of a tile to finish adds them up and sends the sum); a second kernel on each GPU waits for
 * all flags (bounded: 2 s unless set otherwise, then status bit 32 and nothing is stored), adds the partial sums in rank
 * order and rounds once, so every GPU ends with the same bits.  In the normal call the second kernel depends on the flags
 * alone, not on the first kernel having drained; C is complete, as for any call, when the stream reaches the work
 * enqueued after the call.
 * ---------------------------------------------------------------------------------------------------------- */

/* Bytes of one GPU's receive buffer for a group of `world` (1..8) GPUs and outputs of up to `max_elems` = M*N values
 * (a multiple of 4); 0 for bad arguments. */
unsigned long long FlashLLM_Comm_BufferBytes(int world, long long max_elems);

/* Allocates (cudaMalloc) and clears this GPU's receive buffer on the current device; with `ipc_handle` != nullptr also
 * writes the 64-byte inter-process handle (cudaIpcMemHandle_t) other processes open it with. */
int FlashLLM_Comm_AllocBuffer(int world, long long max_elems, void** buffer, void* ipc_handle);
/* Maps a peer's buffer (its 64-byte handle) into this process / unmaps it / frees an own buffer. */
int FlashLLM_Comm_OpenPeerBuffer(const void* ipc_handle, void** buffer);
int FlashLLM_Comm_ClosePeerBuffer(void* buffer);
int FlashLLM_Comm_FreeBuffer(void* buffer);

/* A communicator: `buffers[w]` = GPU w's receive buffer as addressable from this process (`buffers[rank]` the own
 * one).  All GPUs must have allocated (and thereby cleared) their buffers before any of them makes a fused call, and
 * every GPU must make the same sequence of fused calls on its communicator. */
int FlashLLM_Comm_Create(void** comm, int rank, int world, long long max_elems, void* const* buffers);
int FlashLLM_Comm_Destroy(void* comm);
/* How long the summing kernel waits for the slowest GPU of the group before it gives up with status bit 32:
 * 1..60000 ms, 2000 ms unless set.  GPUs enter a layer at slightly different times; the limit only has to end the
 * wait for a partner that never comes. */
int FlashLLM_Comm_SetWaitLimit(void* comm, int milliseconds);

/* C[n][m] = act(sum over the group's GPUs w of sum_k A_w[m][k] * B_w[n][k] + bias[m]) + residual[n][m] on every GPU
 * (`residual`: this GPU's copy of the layer input, or nullptr).  Arguments as FlashLLM_SpMM_SplitK_Epilogue without
 * workspace and Split_K (the library cuts K itself: cluster parts, and up to 8 parts parked in the communicator's
 * buffer).  `phases`: 3 = both kernels (the normal call); 1 = the SpMM and its stores only, 2 = the summing kernel
 * only, ordered after everything enqueued before it -- for a host that drives several GPUs' calls, or several ranks
 * emulated on one GPU, from one thread and wants all sends enqueued before any sum. */
int FlashLLM_SpMM_SplitK_AllReduce(void*       comm,
                                   void*       stream,
                                   const void* Compressed_A,
                                   const int*  TileOffsets,
                                   const void* B,
                                   void*       C,
                                   int         M,
                                   int         N,
                                   int         K,
                                   const void* bias,
                                   int         activation,
                                   const void* residual,
                                   int         phases);

/* SpMM for callers that must not allocate device memory.  (No counterpart in the reference, whose callers always
 * bring a Reduction_Workspace of their own.)  Some hosts of this library cannot call cudaMalloc at the point where
 * they need the product: code running while a CUDA graph is being captured, a serving loop whose memory pool was
 * handed out in full at start-up, a plug-in that is only given input and output buffers.  This entry point is
 * SpMM_SplitK_API with the split-K workspace replaced by an 8 MiB scratch array that is part of the library image:
 * every GPU on which the library is loaded carries it until the process exits.
 *   - Same arguments and results as FlashLLM_SpMM_SplitK, minus `A` and `Reduction_Workspace`.
 *   - Split_K*M*N*2 bytes (what a caller-owned workspace would need) must not exceed 8 MiB; larger requests print
 *     a message to stderr and return cudaErrorInvalidValue.  Split_K = 1 never touches the scratch and is accepted at
 *     any size.
 *   - It calls no cudaMalloc, cudaFree or allocating library routine.  The first call on each device looks up the
 *     scratch's device address (cudaGetSymbolAddress) and raises the kernels' shared-memory limit; make that first
 *     call with the device current and before any stream capture begins.  If that set-up fails, the call returns the
 *     error and the next call tries again.
 *   - All calls on a device share the one scratch array, which keeps the previous call's partial sums; every call
 *     overwrites the part it reads back, so nothing needs clearing, but two calls that overlap on the GPU (different
 *     streams, or graphs replayed concurrently) race on it.  Serialise them, or give the second one a workspace of
 *     its own through FlashLLM_SpMM_SplitK. */
int FlashLLM_SpMM_SplitK_NoAlloc(void*       stream,
                                 const void* Compressed_A,
                                 const int*  TileOffsets,
                                 const void* B,
                                 void*       C,
                                 int         M,
                                 int         N,
                                 int         K,
                                 int         Split_K);

/* Split-K reduction on its own (reference csrc/Reduction_Kernel.cuh:24-45):
 * C[i] = fp16(sum_s float(Workspace[s*M*N + i])). */
int FlashLLM_SplitK_Reduction(void* stream, void* C, const void* Reduction_Workspace, int M, int N, int Split_K);

/* Launch overlap (no counterpart in the reference).  With enable != 0, SpMM kernels are launched with programmatic
 * stream serialisation: a kernel's CTAs may start while the previous kernel of the stream is still draining.  They
 * set up, and stream Compressed_A / TileOffsets, right away; B is read and C / the workspace written only after
 * everything enqueued before has completed.  The caller thereby promises that Compressed_A and TileOffsets of a call
 * are not being produced by work still running in the same stream (weights resident before the calls, the inference
 * case).  Off by default.  Process-wide. */
void FlashLLM_SetLaunchOverlap(int enable);

/* Tuning hook replacing the reference's compile-time TilingConfig<...> choice (csrc/TilingConfig.h:36-52,
 * csrc/SpMM_API.cu:79-118): fixes launch-plan fields for subsequent calls from this process.  `fields` holds up to
 * eleven ints, 0 = choose automatically, in this order:
 *   0 cluster_k       K parts summed inside a thread-block cluster through distributed shared memory (1..8)
 *   1 workspace_k     extra K parts through Reduction_Workspace (capped at Split_K/2 of the call: an fp32 partial
 *                     matrix takes the room of two fp16 ones)
 *   2 a_stages        decompressed 128x64 tiles in flight        3 b_stages  B batches in flight
 *   4 b_batch         K tiles of B per TMA instruction
 *   5 ring_slots x 6 chunk_vectors (16 bytes each, power of two): the compressed-stream ring (ring form only)
 *   7 scatter_warps   warps that decompress tiles, one whole tile per warp at a time (ring form: 4..12, at most
 *                     a_stages; register-streaming form: 4, two CTAs per SM, or 8, one CTA per SM)
 *   8 producers       ring form: warps issuing the bulk copies (1..4; must divide ring_slots); register-streaming form
 *                     with 4 scatter_warps: 2 = two warps share every tile (8 scatter warps on 4 stages)
 *   9 path            1 = ring form: the compressed stream is copied into a shared-memory ring by bulk copies;
 *                     2 = register-streaming form (the default): scatter warps load their tiles' words from global
 *                     memory into registers, tiles alternate between two MMA-issuing threads
 *  10 reduce          who adds the workspace parts up: 1 = a second kernel (the default; with launch overlap it
 *                     hides behind the neighbouring SpMMs); 2 = the SpMM kernel itself: every CTA parks its fp32
 *                     partial tile and counts itself in on a counter of the output tile, the CTA that completes the
 *                     count adds the parts in part order and finishes the output (nobody waits; same bits as 1; the
 *                     counters belong to the library, one set per stream, 32 streams per device -- a 33rd stream, or a
 *                     call with more than 2048 output tiles, gets the second kernel).  The fused all-reduce always
 *                     uses 2 for its own K split.
 * FlashLLM_SetPlan(nullptr, 0) restores automatic choice. */
void FlashLLM_SetPlan(const int* fields, int count);

/* Describes the plan the next SpMM call with these sizes would use: out[0..10] as above, out[11] = dynamic shared
 * memory in bytes; `count` = entries available in `out`. */
int FlashLLM_GetPlan(int M, int N, int K, int Split_K, int* out, int count);

/* Reads and clears the device-side status word of the current device (synchronises the device).  0 = no kernel of
 * this library gave up on a bounded wait or met a malformed TileOffsets since the last call.  Bits: 1 a bounded wait
 * inside a kernel ran out, 2 malformed TileOffsets (nothing stored for that tile row), 8 device encoder: offsets do not
 * match the matrix, 16 misaligned shared memory, 32 fused all-reduce: a GPU of the group did not deliver in time.  A
 * give-up belongs to the launch it happened in: later calls run normally whether or not the word is read. */
unsigned int FlashLLM_ConsumeStatus(void);

/* Number of kernels this library has launched from this process (all devices). */
unsigned long long FlashLLM_LaunchCount(void);

}  // extern "C"
