"""Full-size configurations of the benchmark specification, checked through properties that do not need the whole
product on the CPU: row blocks against the host GEMM, linearity in B, and agreement between two different K splits."""
import numpy as np
import pytest
import torch

from helpers import assert_close

pytestmark = pytest.mark.gpu


def _setup(lib, M, K, N, sparsity, seed):
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    A = lib.synthetic.sparse_uniform_matrix(M, K, sparsity, seed, device=dev)
    mk = lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device=dev))  # noqa: E731
    comp, offs, _, _ = lib.encode_on_device(stream, A.data_ptr(), M, K, mk, mk, lambda o, i: o[i].item())
    B = lib.synthetic.dense_uniform_matrix(N, K, seed ^ 0xB, device=dev)
    return A, B, comp, offs


def _spmm(lib, comp, offs, B, M, N, K, split_k, plan=None):
    C = torch.full((N, M), float("nan"), dtype=torch.float16, device="cuda")
    ws = torch.empty((split_k, N, M), dtype=torch.float16, device="cuda")
    lib.set_plan(**(plan or {}))
    try:
        lib.SpMM_SplitK_API(torch.cuda.current_stream().cuda_stream, None, comp.data_ptr(), offs.data_ptr(), B.data_ptr(),
                            C.data_ptr(), M, N, K, ws.data_ptr(), split_k)
        torch.cuda.synchronize()
    finally:
        lib.set_plan()
    assert lib.consume_status() == 0
    return C


@pytest.mark.parametrize("M,K,N,sparsity,split_k", [
    (36864, 9216, 16, 0.8, 3),      # OPT-66B FFN1
    (9216, 36864, 32, 0.7, 6),      # OPT-66B FFN2
    (27648, 9216, 8, 0.9, 2),       # OPT-66B QKV
    (49152, 12288, 64, 0.8, 9),     # OPT-175B FFN1
    (12288, 49152, 8, 0.9, 8),      # split-K stress
    (2048, 32768, 16, 0.7, 8),      # small M, long K
    (4608, 12288, 16, 0.8, 1),      # 8-way row shard of 36864 x 12288
])
def test_full_size_row_blocks_and_properties(lib, oracle, M, K, N, sparsity, split_k):
    A, B, comp, offs = _setup(lib, M, K, N, sparsity, seed=M + K + N)
    C = _spmm(lib, comp, offs, B, M, N, K, split_k)
    got = C.cpu().numpy()
    assert not np.isnan(got).any()
    # three row blocks against the host GEMM (first, a middle one, last)
    A_h = None
    for r0 in (0, (M // 2 // 128) * 128, M - 128):
        rows = A[r0:r0 + 128].cpu().numpy()
        want = oracle.gemm_f32(rows, B.cpu().numpy())
        assert_close(got[:, r0:r0 + 128], want, f"rows {r0}..{r0 + 128}")
    del A_h
    # a different K split must agree (cluster sum vs workspace sum vs none)
    other = _spmm(lib, comp, offs, B, M, N, K, 8, plan=dict(cluster_k=2, workspace_k=2)).cpu().numpy()
    assert_close(other, got.astype(np.float32), "K split 2x2 vs automatic")
    # linearity: SpMM(2 B) == 2 SpMM(B) exactly -- powers of two commute with every rounding step, except where the
    # fp16 result is subnormal (fixed spacing 2^-24 there), so those few outputs only have to agree to one spacing
    twice = _spmm(lib, comp, offs, (B * 2).contiguous(), M, N, K, split_k).cpu().numpy()
    normal = np.abs(got) >= np.float16(2.0 ** -13)
    assert np.array_equal(twice[normal], (got * np.float16(2))[normal])
    assert np.all(np.abs(twice[~normal].astype(np.float32) - 2 * got[~normal].astype(np.float32)) <= 2.0 ** -23)
