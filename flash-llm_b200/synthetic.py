"""Seeded synthetic inputs with the shapes and value distributions of the SpMM benchmark configurations.

Counter-based (splitmix64 of ``seed`` and the element index), so an element's value depends on nothing but
``(seed, row, column)``: the same matrix comes out on CPU and GPU, in one piece or in row blocks.  These stand
in for pruned OPT weights, as the reference's own benchmark does with random matrices
(Flash-LLM kernel_benchmark/spmm_test_utils.h:103-118).
"""
from __future__ import annotations

import torch

_GOLDEN = 0x9E3779B97F4A7C15 - (1 << 64)
_C1 = 0xBF58476D1CE4E5B9 - (1 << 64)
_C2 = 0x94D049BB133111EB - (1 << 64)


def _lsr(z: torch.Tensor, s: int) -> torch.Tensor:
    return (z >> s) & ((1 << (64 - s)) - 1)


def _mix(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _C1
    z = (z ^ _lsr(z, 27)) * _C2
    return z ^ _lsr(z, 31)


def _to_i64(v: int) -> int:
    v &= (1 << 64) - 1
    return v - (1 << 64) if v >= (1 << 63) else v


def uniform01(seed: int, start: int, count: int, device, stream_id: int = 0) -> torch.Tensor:
    """``count`` float32 values in [0, 1) (24-bit resolution) for element indices ``start .. start+count``."""
    idx = torch.arange(start + 1, start + 1 + count, dtype=torch.int64, device=device)
    z = _mix(idx * _GOLDEN + _to_i64(seed + stream_id * 0x632BE59BD9B4E019))
    return _lsr(z, 40).to(torch.float32) * (1.0 / (1 << 24))


def sparse_uniform_matrix(M: int, K: int, sparsity: float, seed: int, device="cpu", rows_per_block: int = 2048,
                          rows: tuple[int, int] | None = None):
    """fp16 ``[M][K]``: Bernoulli(1 - sparsity) mask, non-zeros U(-1, 1) (never rounding to zero).
    ``rows=(r0, r1)`` returns only that row range of the same matrix (a row shard)."""
    lo, hi = rows if rows is not None else (0, M)
    out = torch.empty((hi - lo, K), dtype=torch.float16, device=device)
    for r0 in range(lo, hi, rows_per_block):
        r1 = min(hi, r0 + rows_per_block)
        n = (r1 - r0) * K
        keep = uniform01(seed, r0 * K, n, device, 0) >= sparsity
        val = uniform01(seed, r0 * K, n, device, 1) * 2.0 - 1.0
        tiny = val.abs() < 6.2e-5
        val = torch.where(tiny, torch.where(val < 0, -6.2e-5, 6.2e-5).to(val.dtype), val)
        out[r0 - lo:r1 - lo] = torch.where(keep, val, torch.zeros_like(val)).to(torch.float16).view(r1 - r0, K)
    return out


def dense_uniform_matrix(N: int, K: int, seed: int, device="cpu") -> torch.Tensor:
    """fp16 ``[N][K]`` with entries U(-1, 1) (the activation matrix B)."""
    return (uniform01(seed, 0, N * K, device, 2) * 2.0 - 1.0).to(torch.float16).view(N, K)


def normal_matrix(M: int, K: int, std: float, seed: int, device="cpu", rows_per_block: int = 2048) -> torch.Tensor:
    """fp32 ``[M][K]`` with entries N(0, std^2) (Box-Muller on the counter streams)."""
    out = torch.empty((M, K), dtype=torch.float32, device=device)
    for r0 in range(0, M, rows_per_block):
        r1 = min(M, r0 + rows_per_block)
        n = (r1 - r0) * K
        u1 = uniform01(seed, r0 * K, n, device, 3).clamp_min(1.0 / (1 << 24))
        u2 = uniform01(seed, r0 * K, n, device, 4)
        out[r0:r1] = (std * torch.sqrt(-2.0 * torch.log(u1)) * torch.cos(6.283185307179586 * u2)).view(r1 - r0, K)
    return out


def magnitude_pruned_matrix(M: int, K: int, sparsity: float, std: float, seed: int, device="cpu") -> torch.Tensor:
    """fp16 ``[M][K]``: N(0, std^2) weights with the smallest ``sparsity`` fraction by magnitude set to zero."""
    w = normal_matrix(M, K, std, seed, device).to(torch.float16)
    drop = int(round(sparsity * M * K))
    if drop > 0:
        mag = w.abs().float().flatten()
        threshold = torch.kthvalue(mag, drop).values if mag.device.type == "cpu" else torch.sort(mag).values[drop - 1]
        w = torch.where(w.abs().float() <= threshold, torch.zeros_like(w), w)
    return w


def reference_style_inputs(M: int, K: int, N: int, sparsity_percent: int, seed: int, device="cpu"):
    """The reference benchmark's degenerate inputs: every kept weight is 1.0 and B takes the five values
    {-0.5, -0.3, -0.1, 0.1, 0.3} (Flash-LLM kernel_benchmark/spmm_test_utils.h:106-117)."""
    r = (uniform01(seed, 0, M * K, device, 5) * 100.0).floor()
    A = (r >= sparsity_percent).to(torch.float16).view(M, K)
    b = (uniform01(seed, 0, N * K, device, 6) * 5.0).floor() / 5.0 - 0.5
    return A, b.to(torch.float16).view(N, K)
