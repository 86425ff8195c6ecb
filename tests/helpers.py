"""Shared helpers of the parity tests: run the product path through its C ABI on device buffers owned by
torch, and compare against the CPU oracle with the tolerance the benchmark specification states."""
from __future__ import annotations

import numpy as np
import torch

# Tolerance of the SpMM parity tests (fp16 outputs, fp32 accumulation): the specification asks for a maximum
# relative error of 1e-2 against the reference; entries much smaller than the typical output magnitude are
# measured against 5 % of the RMS instead of their own value, and the largest absolute error must stay
# below 2e-3 of the largest output.
REL_TOL = 1e-2
ABS_TOL_OF_MAX = 2e-3


def error_metrics(got: np.ndarray, want: np.ndarray) -> tuple[float, float]:
    got = got.astype(np.float64)
    want = want.astype(np.float64)
    finite = np.isfinite(want)
    if not finite.all():  # infinities / NaNs must appear in the same places
        assert np.array_equal(np.isnan(got), np.isnan(want))
        assert np.array_equal(got[np.isinf(want)], want[np.isinf(want)])
        got, want = got[finite], want[finite]
    if want.size == 0:
        return 0.0, 0.0
    rms = float(np.sqrt(np.mean(want * want)))
    floor = max(0.05 * rms, 1e-30)
    rel = float(np.max(np.abs(got - want) / np.maximum(np.abs(want), floor)))
    peak = float(np.max(np.abs(want)))
    ab = float(np.max(np.abs(got - want)) / peak) if peak > 0 else float(np.max(np.abs(got - want)))
    return rel, ab


def assert_close(got: np.ndarray, want: np.ndarray, what: str = "", fp16_partials: int = 0) -> None:
    """``fp16_partials`` = number of fp16-rounded partial sums inside ``want`` (the reference kernel and its CPU
    model round every split-K part to fp16 before adding them, reference csrc/SpMM_Kernel.cuh:385): each adds up to
    half an fp16 ulp of a partial, 2^-11 of the output scale, that no other implementation can reproduce."""
    rel, ab = error_metrics(got, want)
    if fp16_partials:
        w = want.astype(np.float64)
        g = got.astype(np.float64)
        rms = float(np.sqrt(np.mean(w * w)))
        slack = fp16_partials * 2.0 ** -11 * float(np.max(np.abs(w)))
        excess = np.abs(g - w) - slack
        rel = float(np.max(np.maximum(excess, 0.0) / np.maximum(np.abs(w), max(0.05 * rms, 1e-30))))
    assert rel <= REL_TOL and ab <= ABS_TOL_OF_MAX * (1 + fp16_partials), \
        f"{what}: max rel err {rel:.3e}, max abs/peak {ab:.3e}"


class DeviceProblem:
    """Compressed A, B, C and workspace on the GPU for one SpMM; results come back as numpy."""

    def __init__(self, fl, comp: np.ndarray, offs: np.ndarray, B: np.ndarray, M: int, N: int, K: int, split_k: int = 1):
        self.fl, self.M, self.N, self.K, self.split_k = fl, M, N, K, split_k
        dev = torch.device("cuda:0")
        words = comp.view(np.int32) if comp.size else np.zeros(4, np.int32)
        self.comp = torch.from_numpy(np.ascontiguousarray(words)).to(dev)
        self.offs = torch.from_numpy(np.ascontiguousarray(offs.astype(np.int32))).to(dev)
        self.B = torch.from_numpy(np.ascontiguousarray(B.view(np.float16))).to(dev)
        self.C = torch.full((N, M), float("nan"), dtype=torch.float16, device=dev)
        self.ws = torch.empty((max(split_k, 1), N, M), dtype=torch.float16, device=dev)

    def run(self, check_status: bool = True) -> np.ndarray:
        self.C.fill_(float("nan"))
        stream = torch.cuda.current_stream().cuda_stream
        self.fl.SpMM_SplitK_API(stream, None, self.comp.data_ptr(), self.offs.data_ptr(), self.B.data_ptr(),
                                self.C.data_ptr(), self.M, self.N, self.K, self.ws.data_ptr(), self.split_k)
        torch.cuda.synchronize()
        if check_status:
            status = self.fl.consume_status()
            assert status == 0, f"kernel status word {status:#x}"
        return self.C.cpu().numpy()


def random_problem(fl, M: int, K: int, N: int, sparsity: float, seed: int):
    """Seeded inputs as numpy: A[M][K] fp16 (sparse), B[N][K] fp16."""
    A = fl.synthetic.sparse_uniform_matrix(M, K, sparsity, seed).numpy()
    B = fl.synthetic.dense_uniform_matrix(N, K, seed ^ 0xB).numpy()
    return A, B


def assert_close_device(got: torch.Tensor, want: torch.Tensor, what: str = "", fp16_partials: int = 0) -> None:
    """:func:`assert_close` for two device tensors of the same shape, evaluated on the device (whole outputs of the
    full-size configurations: nothing is copied to the host but the two error figures)."""
    assert got.shape == want.shape, f"{what}: shapes {tuple(got.shape)} vs {tuple(want.shape)}"
    g, w = got.double(), want.double()
    assert bool(torch.isfinite(w).all()) and bool(torch.isfinite(g).all()), f"{what}: non-finite outputs"
    rms = float(torch.sqrt(torch.mean(w * w)))
    peak = float(w.abs().max())
    floor = max(0.05 * rms, 1e-30)
    diff = (g - w).abs()
    ab = float(diff.max()) / peak if peak > 0 else float(diff.max())
    excess = torch.clamp(diff - fp16_partials * 2.0 ** -11 * peak, min=0.0) if fp16_partials else diff
    rel = float((excess / torch.clamp(w.abs(), min=floor)).max())
    assert rel <= REL_TOL and ab <= ABS_TOL_OF_MAX * (1 + fp16_partials), \
        f"{what}: max rel err {rel:.3e}, max abs/peak {ab:.3e}"
