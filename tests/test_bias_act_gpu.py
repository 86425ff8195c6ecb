"""The fused output epilogue (bias of the output feature, ReLU, residual) of FlashLLM_SpMM_SplitK_BiasAct and
FlashLLM_SpMM_SplitK_Epilogue against the host: act(GEMM + bias) + residual computed in fp32 and rounded once.  Every way the library finishes an output is covered: the
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


@pytest.mark.parametrize("path", [1, 2], ids=["ring", "direct"])
@pytest.mark.parametrize("plan", PLANS, ids=["plain", "cluster", "workspace", "both"])
@pytest.mark.parametrize("N", [8, 64, 128])
def test_residual_epilogue(lib, oracle, path, plan, N):
    """add-bias-residual after the attention output projection / second FFN matmul: the residual [N][M] joins the
    fp32 sum after the activation."""
    M, K, split_k = 384, 1024, 4
    A, B = random_problem(lib, M, K, N, 0.8, 400 + N)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    rng = np.random.default_rng(6)
    bias = (rng.standard_normal(M) * 2.0).astype(np.float16)
    residual = (rng.standard_normal((N, M)) * 8.0).astype(np.float16)
    want = np.maximum(oracle.gemm_f32(A, B) + bias.astype(np.float32)[None, :], 0.0) + residual.astype(np.float32)
    dev = torch.device("cuda:0")
    to_dev = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)  # noqa: E731
    comp_d, offs_d, B_d, bias_d, res_d = to_dev(comp.view(np.int32)), to_dev(offs), to_dev(B), to_dev(bias), to_dev(residual)
    C = torch.full((N, M), float("nan"), dtype=torch.float16, device=dev)
    ws = torch.empty((split_k, N, M), dtype=torch.float16, device=dev)
    lib.set_plan(path=path, **plan)
    try:
        lib.spmm_splitk_epilogue(torch.cuda.current_stream().cuda_stream, comp_d.data_ptr(), offs_d.data_ptr(),
                                 B_d.data_ptr(), C.data_ptr(), M, N, K, ws.data_ptr(), split_k, bias_d.data_ptr(),
                                 lib.ACT_RELU, res_d.data_ptr())
        torch.cuda.synchronize()
    finally:
        lib.set_plan()
    assert lib.consume_status() == 0
    assert_close(C.cpu().numpy(), want, f"path={path} plan={plan} N={N}")
    assert torch.equal(res_d.cpu(), torch.from_numpy(residual))  # the residual is only read


def test_residual_overlapping_the_output_is_refused(lib):
    assert lib.library().FlashLLM_SpMM_SplitK_Epilogue(None, 0x1000, 0x1000, 0x1000, 0x2000, 128, 16, 64, None, 1, None, 0,
                                                       0x2000) == 1


def test_unknown_activation_is_refused(lib):
    assert lib.library().FlashLLM_SpMM_SplitK_BiasAct(None, 0x1000, 0x1000, 0x1000, 0x1000, 128, 16, 64, None, 1, None, 7) == 1
