"""The fused output epilogue (bias of the output feature, ReLU) of FlashLLM_SpMM_SplitK_BiasAct against the host:
act(GEMM + bias) computed in fp32 and rounded once.  Every way the library finishes an output is covered: the
kernel's own epilogue, the sum inside a cluster and the sum of workspace parts, in both forms of the kernel."""
import numpy as np
import pytest
import torch

from helpers import assert_close, random_problem

pytestmark = pytest.mark.gpu

PLANS = [dict(cluster_k=1, workspace_k=1), dict(cluster_k=4, workspace_k=1), dict(cluster_k=1, workspace_k=4),
         dict(cluster_k=2, workspace_k=2)]


@pytest.mark.parametrize("path", [1, 2], ids=["ring", "direct"])
@pytest.mark.parametrize("plan", PLANS, ids=["plain", "cluster", "workspace", "both"])
@pytest.mark.parametrize("use_bias,activation", [(True, 1), (True, 0), (False, 1)])
def test_bias_and_relu_epilogue(lib, oracle, path, plan, use_bias, activation):
    M, K, N, split_k = 512, 2048, 16, 8
    A, B = random_problem(lib, M, K, N, 0.8, 300 + path)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    bias = (np.random.default_rng(5).standard_normal(M) * 4.0).astype(np.float16)
    want = oracle.gemm_f32(A, B)
    if use_bias:
        want = want + bias.astype(np.float32)[None, :]
    if activation:
        want = np.maximum(want, 0.0)
    dev = torch.device("cuda:0")
    to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    comp_d, offs_d, B_d, bias_d = to_dev(comp.view(np.int32)), to_dev(offs), to_dev(B), to_dev(bias)
    C = torch.full((N, M), float("nan"), dtype=torch.float16, device=dev)
    ws = torch.empty((split_k, N, M), dtype=torch.float16, device=dev)
    lib.set_plan(path=path, **plan)
    try:
        lib.spmm_splitk_bias_act(torch.cuda.current_stream().cuda_stream, comp_d.data_ptr(), offs_d.data_ptr(),
                                 B_d.data_ptr(), C.data_ptr(), M, N, K, ws.data_ptr(), split_k,
                                 bias_d.data_ptr() if use_bias else None, activation)
        torch.cuda.synchronize()
    finally:
        lib.set_plan()
    assert lib.consume_status() == 0
    got = C.cpu().numpy()
    assert_close(got, want, f"path={path} plan={plan} bias={use_bias} act={activation}")
    if activation:
        assert (got >= 0).all() and (got == 0).any()


def test_unknown_activation_is_refused(lib):
    assert lib.library().FlashLLM_SpMM_SplitK_BiasAct(None, 0x1000, 0x1000, 0x1000, 0x1000, 128, 16, 64, None, 1, None, 7) == 1
