"""``torch.ops.flashllm``: the library's SpMM as PyTorch operators, for integration tests and for callers whose tensors
live in torch.  Importing this module registers

* ``flashllm::encode(Tensor A) -> (Tensor compressed, Tensor tile_offsets)``: a dense fp16 weight ``A[M][K]`` on a CUDA
  device to its tiled-CSL form (int32 words, int32 tile offsets) with the device encoder; what the reference does on
  the host with ``InitSparseMatrixA_API`` (reference csrc/SpMM_API.cu:449-494).
* ``flashllm::spmm(Tensor compressed, Tensor tile_offsets, Tensor B, int M, int split_k=1) -> Tensor``:
  ``C[N][M] = B[N][K] @ A[M][K]^T`` (reference ``SpMM_SplitK_API``, csrc/SpMM_API.cu:124-171).
* ``flashllm::spmm_epilogue(..., Tensor? bias, int activation, Tensor? residual) -> Tensor``: the same with
  ``act(. + bias[M]) + residual[N][M]`` applied to the fp32 sums before the one rounding.

The operators run on the current CUDA stream of B's device and call the library through its C ABI; there is no CPU
implementation (a CPU tensor is refused), only shape inference for meta tensors.
"""
from __future__ import annotations

import torch

from . import api

_LIB = torch.library.Library("flashllm", "DEF")
_LIB.define("encode(Tensor A) -> (Tensor, Tensor)")
_LIB.define("spmm(Tensor compressed, Tensor tile_offsets, Tensor B, int M, int split_k=1) -> Tensor")
_LIB.define("spmm_epilogue(Tensor compressed, Tensor tile_offsets, Tensor B, int M, int split_k=1, Tensor? bias=None, "
            "int activation=0, Tensor? residual=None) -> Tensor")


def _check_operands(compressed: torch.Tensor, tile_offsets: torch.Tensor, B: torch.Tensor, M: int) -> tuple[int, int]:
    if not B.is_cuda:
        raise RuntimeError("flashllm::spmm runs on CUDA tensors only")
    if B.dtype != torch.float16 or B.dim() != 2 or not B.is_contiguous():
        raise RuntimeError("B must be a contiguous fp16 matrix [N][K]")
    if compressed.dtype != torch.int32 or tile_offsets.dtype != torch.int32:
        raise RuntimeError("compressed and tile_offsets must be int32 tensors (tiled-CSL words, offsets in vectors)")
    if compressed.device != B.device or tile_offsets.device != B.device:
        raise RuntimeError("all operands must live on one device")
    N, K = B.shape
    if M % 128 or K % 64:
        raise RuntimeError(f"M ({M}) must be a multiple of 128 and K ({K}) of 64")
    if tile_offsets.numel() != (M // 128) * (K // 64) + 2:
        raise RuntimeError("tile_offsets does not belong to an M x K matrix of this shape")
    return N, K


def _run(compressed, tile_offsets, B, M, split_k, bias, activation, residual) -> torch.Tensor:
    N, K = _check_operands(compressed, tile_offsets, B, M)
    for name, t, shape in (("bias", bias, (M,)), ("residual", residual, (N, M))):
        if t is not None and (t.dtype != torch.float16 or tuple(t.shape) != shape or not t.is_contiguous()
                              or t.device != B.device):
            raise RuntimeError(f"{name} must be a contiguous fp16 tensor of shape {shape} on B's device")
    with torch.cuda.device(B.device):
        C = torch.empty((N, M), dtype=torch.float16, device=B.device)
        # the room the reference's callers bring: Split_K fp16 matrices (reference csrc/SpMM_API.cu:150-152)
        workspace = torch.empty((split_k, N, M), dtype=torch.float16, device=B.device) if split_k > 1 else None
        api.spmm_splitk_epilogue(torch.cuda.current_stream().cuda_stream, compressed.data_ptr(), tile_offsets.data_ptr(),
                                 B.data_ptr(), C.data_ptr(), M, N, K, workspace.data_ptr() if split_k > 1 else None,
                                 split_k, None if bias is None else bias.data_ptr(), activation,
                                 None if residual is None else residual.data_ptr())
    return C


def _encode_cuda(A: torch.Tensor):
    if A.dtype != torch.float16 or A.dim() != 2 or not A.is_contiguous():
        raise RuntimeError("A must be a contiguous fp16 matrix [M][K]")
    M, K = A.shape
    if M % 128 or K % 64:
        raise RuntimeError(f"M ({M}) must be a multiple of 128 and K ({K}) of 64")
    with torch.cuda.device(A.device):
        stream = torch.cuda.current_stream()

        def alloc(n):
            t = torch.empty(n, dtype=torch.int32, device=A.device)
            return t, t.data_ptr()

        def read(t, i):
            stream.synchronize()
            return int(t[i].item())

        comp, offs, _, words = api.encode_on_device(stream.cuda_stream, A.data_ptr(), M, K, alloc, alloc, read)
    return comp[:words], offs


def _spmm_cuda(compressed, tile_offsets, B, M, split_k=1):
    return _run(compressed, tile_offsets, B, M, split_k, None, api.ACT_NONE, None)


def _spmm_epilogue_cuda(compressed, tile_offsets, B, M, split_k=1, bias=None, activation=0, residual=None):
    return _run(compressed, tile_offsets, B, M, split_k, bias, activation, residual)


def _refuse_cpu(*args, **kwargs):
    raise RuntimeError("flashllm operators have no CPU implementation: move the tensors to a CUDA device")


_LIB.impl("encode", _encode_cuda, "CUDA")
_LIB.impl("spmm", _spmm_cuda, "CUDA")
_LIB.impl("spmm_epilogue", _spmm_epilogue_cuda, "CUDA")
for _name in ("encode", "spmm", "spmm_epilogue"):
    _LIB.impl(_name, _refuse_cpu, "CPU")


@torch.library.register_fake("flashllm::spmm")
def _spmm_fake(compressed, tile_offsets, B, M, split_k=1):
    return B.new_empty((B.shape[0], M))


@torch.library.register_fake("flashllm::spmm_epilogue")
def _spmm_epilogue_fake(compressed, tile_offsets, B, M, split_k=1, bias=None, activation=0, residual=None):
    return B.new_empty((B.shape[0], M))


def spmm(compressed: torch.Tensor, tile_offsets: torch.Tensor, B: torch.Tensor, M: int, split_k: int = 1) -> torch.Tensor:
    """Python spelling of ``torch.ops.flashllm.spmm``."""
    return torch.ops.flashllm.spmm(compressed, tile_offsets, B, M, split_k)
