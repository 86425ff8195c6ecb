"""ctypes host side of ``libSpMM_API.so``, mirroring the reference's operator interface
(Flash-LLM build/SpMM_API.cuh:38-67): same names, argument order and meaning.

Device buffers are passed as integer device pointers (e.g. ``tensor.data_ptr()``); torch is only the
owner of device memory and streams in the callers, never part of a signature here.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_PKG = os.path.dirname(os.path.abspath(__file__))
_ROOT = os.path.dirname(_PKG)
# FLASHLLM_LIBRARY selects another build of the same library (e.g. a pipeline-analysis build).
LIBRARY_PATH = os.environ.get("FLASHLLM_LIBRARY") or os.path.join(_ROOT, "build", "libSpMM_API.so")

_u32p = C.POINTER(C.c_uint32)
_i32p = C.POINTER(C.c_int)


class FlashLLMError(RuntimeError):
    """A library call returned a CUDA error code or the library is unavailable."""


def build_library(verbose: bool = False) -> str:
    """Compile ``build/libSpMM_API.so`` for sm_100a with nvcc (no GPU needed)."""
    cmd = ["make", "-C", os.path.join(_PKG, "csrc")] + ([] if verbose else ["-s"])
    subprocess.run(cmd, check=True)
    return LIBRARY_PATH


_lib = None


def library() -> C.CDLL:
    """The loaded library; raises :class:`FlashLLMError` when it has not been built."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIBRARY_PATH):
        raise FlashLLMError(
            f"{LIBRARY_PATH} is missing: build it with `make -C flash-llm_b200/csrc` "
            "(or __graft_entry__.build()); there is no fallback implementation")
    L = C.CDLL(LIBRARY_PATH)
    L.FlashLLM_SpMM_SplitK.restype = C.c_int
    L.FlashLLM_SpMM_SplitK.argtypes = [C.c_void_p] * 3 + [C.c_void_p] * 3 + [C.c_int] * 3 + [C.c_void_p, C.c_int]
    L.FlashLLM_SpMM_SplitK_BiasAct.restype = C.c_int
    L.FlashLLM_SpMM_SplitK_BiasAct.argtypes = ([C.c_void_p] * 5 + [C.c_int] * 3 + [C.c_void_p, C.c_int, C.c_void_p, C.c_int])
    L.FlashLLM_SpMM_SplitK_Epilogue.restype = C.c_int
    L.FlashLLM_SpMM_SplitK_Epilogue.argtypes = ([C.c_void_p] * 5 + [C.c_int] * 3
                                                + [C.c_void_p, C.c_int, C.c_void_p, C.c_int, C.c_void_p])
    for name in ("FlashLLM_InitSparseMatrixA", "FlashLLM_InitSparseMatrixA_NoReorder"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [C.c_void_p, C.c_int, C.c_int, C.c_int, C.POINTER(_u32p), C.POINTER(_i32p)]
    L.FlashLLM_Free.argtypes = [C.c_void_p]
    L.GenSparseMatrixBinFile.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_char_p, C.c_char_p, C.c_char_p]
    L.FlashLLM_EncodeOnDevice_TileOffsets.restype = C.c_int
    L.FlashLLM_EncodeOnDevice_TileOffsets.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p]
    L.FlashLLM_EncodeOnDevice_Pack.restype = C.c_int
    L.FlashLLM_EncodeOnDevice_Pack.argtypes = [C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p,
                                               C.c_int]
    L.FlashLLM_GenSparseMatrixBinFile_Device.restype = C.c_int
    L.FlashLLM_GenSparseMatrixBinFile_Device.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_char_p, C.c_char_p, C.c_char_p]
    L.FlashLLM_ReadOutputSizes.restype = C.c_int
    L.FlashLLM_ReadOutputSizes.argtypes = [C.c_char_p, _i32p, _i32p]
    L.FlashLLM_ReadSparseMatrixBinFiles.restype = C.c_int
    L.FlashLLM_ReadSparseMatrixBinFiles.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    L.FlashLLM_LoadSparseMatrixBinFiles.restype = C.c_int
    L.FlashLLM_LoadSparseMatrixBinFiles.argtypes = [C.c_char_p, C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p]
    for name in ("FlashLLM_WriteRankLists", "FlashLLM_ReadRankLists"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [C.c_char_p, C.c_int, C.c_int, C.c_void_p, C.c_void_p, C.c_void_p]
    L.FlashLLM_SpMM_SplitK_NoAlloc.restype = C.c_int
    L.FlashLLM_SpMM_SplitK_NoAlloc.argtypes = [C.c_void_p] * 5 + [C.c_int] * 4
    L.FlashLLM_Comm_BufferBytes.restype = C.c_ulonglong
    L.FlashLLM_Comm_BufferBytes.argtypes = [C.c_int, C.c_longlong]
    L.FlashLLM_Comm_AllocBuffer.restype = C.c_int
    L.FlashLLM_Comm_AllocBuffer.argtypes = [C.c_int, C.c_longlong, C.POINTER(C.c_void_p), C.c_void_p]
    L.FlashLLM_Comm_OpenPeerBuffer.restype = C.c_int
    L.FlashLLM_Comm_OpenPeerBuffer.argtypes = [C.c_void_p, C.POINTER(C.c_void_p)]
    for name in ("FlashLLM_Comm_ClosePeerBuffer", "FlashLLM_Comm_FreeBuffer", "FlashLLM_Comm_Destroy"):
        f = getattr(L, name)
        f.restype = C.c_int
        f.argtypes = [C.c_void_p]
    L.FlashLLM_Comm_SetWaitLimit.restype = C.c_int
    L.FlashLLM_Comm_SetWaitLimit.argtypes = [C.c_void_p, C.c_int]
    L.FlashLLM_Comm_Create.restype = C.c_int
    L.FlashLLM_Comm_Create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_int, C.c_longlong, C.POINTER(C.c_void_p)]
    L.FlashLLM_SpMM_SplitK_AllReduce.restype = C.c_int
    L.FlashLLM_SpMM_SplitK_AllReduce.argtypes = [C.c_void_p] * 6 + [C.c_int] * 3 + [C.c_void_p, C.c_int, C.c_void_p, C.c_int]
    L.FlashLLM_SplitK_Reduction.restype = C.c_int
    L.FlashLLM_SplitK_Reduction.argtypes = [C.c_void_p, C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_int]
    L.FlashLLM_SetLaunchOverlap.argtypes = [C.c_int]
    L.FlashLLM_SetPlan.argtypes = [_i32p, C.c_int]
    L.FlashLLM_GetPlan.restype = C.c_int
    L.FlashLLM_GetPlan.argtypes = [C.c_int] * 4 + [_i32p, C.c_int]
    L.FlashLLM_ConsumeStatus.restype = C.c_uint
    L.FlashLLM_LaunchCount.restype = C.c_ulonglong
    _lib = L
    return L


def _check(code: int, what: str) -> None:
    if code != 0:
        raise FlashLLMError(f"{what} failed with cudaError_t {code}")


# ----------------------------------------------------------------------------- encoders (host)

def _encode_host(A_h: np.ndarray, reorder: bool) -> tuple[np.ndarray, np.ndarray, int]:
    if A_h.dtype == np.float16:
        A_h = A_h.view(np.uint16)
    if A_h.dtype != np.uint16 or A_h.ndim != 2:
        raise TypeError("A_h must be a 2-D float16 (or uint16 bit pattern) array")
    A_h = np.ascontiguousarray(A_h)
    M, K = A_h.shape
    L = library()
    fn = L.FlashLLM_InitSparseMatrixA if reorder else L.FlashLLM_InitSparseMatrixA_NoReorder
    comp_p, offs_p = _u32p(), _i32p()
    n = fn(A_h.ctypes.data, M, 0, K, C.byref(comp_p), C.byref(offs_p))
    if n < 0:
        raise FlashLLMError({-1: f"M={M} must be a positive multiple of 128 and K={K} of 64",
                             -2: "out of host memory", -3: "matrix too large for 32-bit TileOffsets"}.get(n, str(n)))
    offs = np.ctypeslib.as_array(offs_p, shape=(n,)).copy()
    words = int(offs[-1]) * 4
    comp = np.ctypeslib.as_array(comp_p, shape=(max(words, 1),))[:words].copy()
    L.FlashLLM_Free(C.cast(comp_p, C.c_void_p))
    L.FlashLLM_Free(C.cast(offs_p, C.c_void_p))
    return comp, offs, n


def InitSparseMatrixA_API(A_h: np.ndarray, M: int | None = None, N: int = 0, K: int | None = None):
    """Dense fp16 ``A_h[M][K]`` -> ``(Compressed_A uint32[NNZ], TileOffsets int32[NumOffsets], NumOffsets)``,
    bit-identical to the reference encoder (csrc/SpMM_API.cu:163-360).  ``N`` is ignored, as there."""
    del N
    if M is not None and K is not None:
        A_h = np.asarray(A_h).reshape(M, K)
    return _encode_host(A_h, True)


def InitSparseMatrixA_API_NoReorder(A_h: np.ndarray, M: int | None = None, N: int = 0, K: int | None = None):
    """Scan-order variant (reference csrc/SpMM_API.cu:363-489)."""
    del N
    if M is not None and K is not None:
        A_h = np.asarray(A_h).reshape(M, K)
    return _encode_host(A_h, False)


def GenSparseMatrixBinFile(dense_file: str, M: int, K: int, nz_weights_file: str, tile_offsets_file: str,
                           output_sizes_file: str) -> None:
    """File-to-file conversion (reference csrc/SpMM_API.cu:500-555), byte-compatible outputs."""
    library().GenSparseMatrixBinFile(dense_file.encode(), M, K, nz_weights_file.encode(), tile_offsets_file.encode(),
                                     output_sizes_file.encode())


_FILE_ERRORS = {-1: "a file cannot be opened or created", -2: "a file is shorter than asked for",
                -3: "the contents are not a well-formed tiled-CSL matrix", -4: "bad arguments"}


def _check_file(code: int, what: str) -> None:
    if code != 0:
        raise FlashLLMError(f"{what}: {_FILE_ERRORS.get(code, f'cudaError_t {code}')}")


def gen_sparse_matrix_bin_file_device(dense_file: str, M: int, K: int, nz_weights_file: str, tile_offsets_file: str,
                                      output_sizes_file: str) -> None:
    """``GenSparseMatrixBinFile`` with the encoding done on the current CUDA device; byte-identical output files."""
    _check_file(library().FlashLLM_GenSparseMatrixBinFile_Device(
        dense_file.encode(), M, K, nz_weights_file.encode(), tile_offsets_file.encode(), output_sizes_file.encode()),
        "GenSparseMatrixBinFile_Device")


def read_output_sizes(output_sizes_file: str) -> tuple[int, int]:
    """``(NNZ, NumOffsets)`` of an ``.OutputSizes.bin`` file (reference csrc/SpMM_API.cu:536-541)."""
    nnz, num_offsets = C.c_int(), C.c_int()
    _check_file(library().FlashLLM_ReadOutputSizes(output_sizes_file.encode(), C.byref(nnz), C.byref(num_offsets)),
                f"read {output_sizes_file}")
    return nnz.value, num_offsets.value


def read_sparse_matrix_bin_files(nz_weights_file: str, tile_offsets_file: str, nnz: int, num_offsets: int):
    """The words and offsets of a converted matrix as numpy arrays, validated (the host half of FasterTransformer's
    ``loadDataArrayFromBin``, reference third_party/ft.patch:3743-3790)."""
    comp = np.empty(max(nnz, 1), np.uint32)
    offs = np.empty(num_offsets, np.int32)
    _check_file(library().FlashLLM_ReadSparseMatrixBinFiles(nz_weights_file.encode(), tile_offsets_file.encode(), nnz,
                                                            num_offsets, comp.ctypes.data, offs.ctypes.data),
                f"read {nz_weights_file} / {tile_offsets_file}")
    return comp[:nnz], offs


def load_sparse_matrix_bin_files(nz_weights_file: str, tile_offsets_file: str, nnz: int, num_offsets: int,
                                 Compressed_A_d: int, TileOffsets_d: int) -> None:
    """The same into device buffers (integer device pointers) of the caller, ready for ``SpMM_SplitK_API``."""
    _check_file(library().FlashLLM_LoadSparseMatrixBinFiles(nz_weights_file.encode(), tile_offsets_file.encode(), nnz,
                                                            num_offsets, Compressed_A_d, TileOffsets_d),
                f"load {nz_weights_file} / {tile_offsets_file}")


def write_rank_lists(model_dir: str, rank: int, nnz_list, num_offsets_list, split_k_list) -> None:
    """``NNZ_List.<rank>.bin``, ``NumOffsets_List.<rank>.bin``, ``SplitK_List.<rank>.bin`` (reference
    end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:188-195)."""
    a, b, c = (np.ascontiguousarray(x, dtype=np.int32) for x in (nnz_list, num_offsets_list, split_k_list))
    if not (a.shape == b.shape == c.shape and a.ndim == 1):
        raise TypeError("the three lists must be one-dimensional and of equal length")
    _check_file(library().FlashLLM_WriteRankLists(model_dir.encode(), rank, a.size, a.ctypes.data, b.ctypes.data,
                                                  c.ctypes.data), f"write rank lists of rank {rank}")


def read_rank_lists(model_dir: str, rank: int, entries: int):
    """The three per-rank lists (``entries`` = 4 x decoder layers) as numpy int32 arrays."""
    a, b, c = (np.empty(entries, np.int32) for _ in range(3))
    _check_file(library().FlashLLM_ReadRankLists(model_dir.encode(), rank, entries, a.ctypes.data, b.ctypes.data,
                                                 c.ctypes.data), f"read rank lists of rank {rank}")
    return a, b, c


# ----------------------------------------------------------------------------- device entry points

def SpMM_SplitK_API(stream: int, A: int | None, Compressed_A: int, TileOffsets: int, B: int, C_out: int, M: int,
                    N: int, K: int, Reduction_Workspace: int | None, Split_K: int) -> None:
    """Enqueue ``C[N][M] = B[N][K] @ A[M][K]^T`` on ``stream`` (reference csrc/SpMM_API.cu:55-130).
    All buffer arguments are integer device pointers; ``A`` is unused and may be ``None``."""
    code = library().FlashLLM_SpMM_SplitK(stream, A, Compressed_A, TileOffsets, B, C_out, M, N, K,
                                          Reduction_Workspace, Split_K)
    _check(code, f"SpMM_SplitK_API(M={M}, N={N}, K={K}, Split_K={Split_K})")


ACT_NONE, ACT_RELU = 0, 1


def spmm_splitk_bias_act(stream: int, Compressed_A: int, TileOffsets: int, B: int, C_out: int, M: int, N: int, K: int,
                         Reduction_Workspace: int | None, Split_K: int, bias: int | None = None,
                         activation: int = ACT_NONE) -> None:
    """``C[N][M] = act(B[N][K] @ A[M][K]^T + bias[M])`` with the epilogue applied to the fp32 sums before the one fp16
    rounding; ``bias`` is a device pointer to M halves or ``None``, ``activation`` ``ACT_NONE`` or ``ACT_RELU``."""
    code = library().FlashLLM_SpMM_SplitK_BiasAct(stream, Compressed_A, TileOffsets, B, C_out, M, N, K,
                                                  Reduction_Workspace, Split_K, bias, activation)
    _check(code, f"SpMM_SplitK_BiasAct(M={M}, N={N}, K={K}, Split_K={Split_K})")


def spmm_splitk_epilogue(stream: int, Compressed_A: int, TileOffsets: int, B: int, C_out: int, M: int, N: int, K: int,
                         Reduction_Workspace: int | None, Split_K: int, bias: int | None = None,
                         activation: int = ACT_NONE, residual: int | None = None) -> None:
    """``C[N][M] = act(B @ A^T + bias[M]) + residual[N][M]``, all on the fp32 sums before the one fp16 rounding (the
    add-bias-residual step a decoder layer runs after its attention output projection and its second feed-forward
    matmul).  ``residual`` is a device matrix laid out like C that does not overlap it, or ``None``."""
    code = library().FlashLLM_SpMM_SplitK_Epilogue(stream, Compressed_A, TileOffsets, B, C_out, M, N, K,
                                                   Reduction_Workspace, Split_K, bias, activation, residual)
    _check(code, f"SpMM_SplitK_Epilogue(M={M}, N={N}, K={K}, Split_K={Split_K})")


def spmm_splitk_no_alloc(stream: int, Compressed_A: int, TileOffsets: int, B: int, C_out: int, M: int, N: int, K: int,
                         Split_K: int) -> None:
    """SpMM for callers that may not allocate device memory (graph capture in progress, a fully pre-assigned
    memory pool, a plug-in that only receives its buffers): the split-K scratch is an 8 MiB array inside the
    library instead of a caller workspace.  ``Split_K*M*N*2`` must fit in it.  Calls that overlap on the GPU share
    that array and race; the first call on a device should precede any stream capture."""
    code = library().FlashLLM_SpMM_SplitK_NoAlloc(stream, Compressed_A, TileOffsets, B, C_out, M, N, K, Split_K)
    _check(code, f"SpMM_SplitK_NoAlloc(M={M}, N={N}, K={K}, Split_K={Split_K})")


# ----------------------------------------------------------------------------- fused row-parallel SpMM + all-reduce

IPC_HANDLE_BYTES = 64  # sizeof(cudaIpcMemHandle_t)


def comm_alloc_buffer(world: int, max_elems: int) -> tuple[int, bytes]:
    """This GPU's receive buffer for a group of ``world`` GPUs and outputs of up to ``max_elems`` (= M*N) values:
    ``(device pointer, inter-process handle)``.  The handle is what the other ranks pass to
    :func:`comm_open_peer_buffer`."""
    ptr = C.c_void_p()
    handle = C.create_string_buffer(IPC_HANDLE_BYTES)
    _check(library().FlashLLM_Comm_AllocBuffer(world, max_elems, C.byref(ptr), handle), "Comm_AllocBuffer")
    return int(ptr.value), handle.raw


def comm_open_peer_buffer(handle: bytes) -> int:
    """Maps another rank's receive buffer (its :func:`comm_alloc_buffer` handle) into this process."""
    ptr = C.c_void_p()
    _check(library().FlashLLM_Comm_OpenPeerBuffer(C.create_string_buffer(handle, IPC_HANDLE_BYTES), C.byref(ptr)),
           "Comm_OpenPeerBuffer")
    return int(ptr.value)


def comm_close_peer_buffer(ptr: int) -> None:
    _check(library().FlashLLM_Comm_ClosePeerBuffer(ptr), "Comm_ClosePeerBuffer")


def comm_free_buffer(ptr: int) -> None:
    _check(library().FlashLLM_Comm_FreeBuffer(ptr), "Comm_FreeBuffer")


def comm_create(rank: int, world: int, max_elems: int, buffers: list[int]):
    """A communicator for :func:`spmm_splitk_allreduce`: ``buffers[w]`` is rank w's receive buffer as mapped in this
    process (``buffers[rank]`` the own one).  Every rank must make the same sequence of fused calls on it."""
    comm = C.c_void_p()
    arr = (C.c_void_p * world)(*buffers)
    _check(library().FlashLLM_Comm_Create(C.byref(comm), rank, world, max_elems, arr), "Comm_Create")
    return comm


def comm_set_wait_limit(comm, milliseconds: int) -> None:
    """How long the summing kernel waits for the slowest rank before giving up with status bit 32 (default 2000 ms)."""
    _check(library().FlashLLM_Comm_SetWaitLimit(comm, milliseconds), "Comm_SetWaitLimit")


def comm_destroy(comm) -> None:
    library().FlashLLM_Comm_Destroy(comm)


def spmm_splitk_allreduce(comm, stream: int, Compressed_A: int, TileOffsets: int, B: int, C_out: int, M: int, N: int,
                          K: int, bias: int | None = None, activation: int = ACT_NONE, phases: int = 3,
                          residual: int | None = None) -> None:
    """Row-parallel SpMM with the all-reduce fused in: ``C[N][M] = act(sum over the group of (B_w @ A_w^T) + bias)
    + residual``,
    where this rank holds the K slice ``A_w[M][K]``, ``B_w[N][K]``.  Every rank's kernel stores its fp32 partial sums
    straight into all ranks' receive buffers; a second kernel adds them in rank order and rounds once, so every rank
    ends with the same bits.  ``phases``: 3 = both kernels (the normal call), 1 = the SpMM and its stores only,
    2 = the summing kernel only (for driving several ranks from one stream: all ranks' phase 1, then their phase 2)."""
    code = library().FlashLLM_SpMM_SplitK_AllReduce(comm, stream, Compressed_A, TileOffsets, B, C_out, M, N, K, bias,
                                                    activation, residual, phases)
    _check(code, f"SpMM_SplitK_AllReduce(M={M}, N={N}, K={K})")


def splitk_reduction(stream: int, C_out: int, workspace: int, M: int, N: int, split_k: int) -> None:
    """``C[i] = fp16(sum_s float(workspace[s*M*N + i]))`` (reference csrc/Reduction_Kernel.cuh:24-45)."""
    _check(library().FlashLLM_SplitK_Reduction(stream, C_out, workspace, M, N, split_k), "SplitK_Reduction")


def encode_on_device(stream: int, A_d: int, M: int, K: int, alloc_i32, alloc_u32, read_i32):
    """Device encoder.  ``alloc_i32(n)`` / ``alloc_u32(n)`` return ``(owner, device_pointer)`` for ``n``
    elements of device memory, ``read_i32(owner, index)`` reads one int back after synchronising the stream.
    Returns ``(compressed_owner, offsets_owner, num_offsets, nnz_words)``."""
    T = (M // 128) * (K // 64)
    offs_owner, offs_ptr = alloc_i32(T + 2)
    _check(library().FlashLLM_EncodeOnDevice_TileOffsets(stream, A_d, M, K, offs_ptr), "EncodeOnDevice_TileOffsets")
    words = int(read_i32(offs_owner, T + 1)) * 4
    comp_owner, comp_ptr = alloc_u32(max(words, 4))
    _check(library().FlashLLM_EncodeOnDevice_Pack(stream, A_d, M, K, offs_ptr, comp_ptr, 1), "EncodeOnDevice_Pack")
    return comp_owner, offs_owner, T + 2, words


def set_launch_overlap(enable: bool) -> None:
    """Let consecutive SpMM kernels of a stream overlap (set-up and weight streaming of the next start while the
    previous drains).  Only valid when the compressed weights are not produced by work still running in that stream."""
    library().FlashLLM_SetLaunchOverlap(1 if enable else 0)


PLAN_FIELDS = ("cluster_k", "workspace_k", "a_stages", "b_stages", "b_batch", "ring_slots", "chunk_vectors",
               "scatter_warps", "producers", "path", "reduce")
PATH_RING, PATH_DIRECT = 1, 2
REDUCE_SECOND_KERNEL, REDUCE_LAST_CTA = 1, 2


def set_plan(**fields: int) -> None:
    """Pin launch-plan fields for later calls (absent or 0 = automatic); ``set_plan()`` restores the defaults."""
    unknown = set(fields) - set(PLAN_FIELDS)
    if unknown:
        raise TypeError(f"unknown plan fields {sorted(unknown)}; known: {PLAN_FIELDS}")
    values = (C.c_int * len(PLAN_FIELDS))(*[int(fields.get(name, 0)) for name in PLAN_FIELDS])
    library().FlashLLM_SetPlan(values, len(PLAN_FIELDS))


def get_plan(M: int, N: int, K: int, Split_K: int = 1) -> dict:
    out = (C.c_int * (len(PLAN_FIELDS) + 1))()
    _check(library().FlashLLM_GetPlan(M, N, K, Split_K, out, len(PLAN_FIELDS) + 1), "GetPlan")
    return dict(zip(PLAN_FIELDS + ("smem_bytes",), list(out)))


def consume_status() -> int:
    """Synchronise the device and return-and-clear the kernel status word (0 = healthy)."""
    return int(library().FlashLLM_ConsumeStatus())


def launch_count() -> int:
    return int(library().FlashLLM_LaunchCount())
