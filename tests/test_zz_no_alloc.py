"""The allocation-free SpMM entry point against the ordinary one.

Some callers of this library cannot allocate device memory when they need the product — a CUDA graph is being
captured, the process's memory pool was handed out in full at start-up, or the caller is a plug-in that only ever
sees its input and output buffers.  For them FlashLLM_SpMM_SplitK_NoAlloc keeps the split-K scratch inside the
library.  This file is collected last on purpose: if the new entry point misbehaved, every other test has already
run.  It checks, on two calls in a row (the scratch keeps the first call's partial sums), that the new entry point
gives what FlashLLM_SpMM_SplitK gives with a caller-owned workspace, and that oversized requests are refused.
"""
import numpy as np
import pytest
import torch

from helpers import assert_close, random_problem

pytestmark = pytest.mark.gpu


def _device_problem(lib, M, K, N, sparsity, seed):
    A, B = random_problem(lib, M, K, N, sparsity, seed)
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    dev = torch.device("cuda:0")
    words = comp.view(np.int32) if comp.size else np.zeros(4, np.int32)
    return (A, B, torch.from_numpy(np.ascontiguousarray(words)).to(dev), torch.from_numpy(offs).to(dev),
            torch.from_numpy(B).to(dev))


@pytest.mark.parametrize("M,K,N,split_k", [(256, 2048, 16, 8), (512, 4096, 8, 4), (1024, 1024, 32, 1)])
def test_no_alloc_entry_matches_workspace_entry(lib, oracle, M, K, N, split_k):
    A, B, comp_d, offs_d, B_d = _device_problem(lib, M, K, N, 0.8, seed=7 + N)
    stream = torch.cuda.current_stream().cuda_stream
    if split_k > 1:  # problems this small would be cut inside clusters: pin the cut that goes through the scratch
        lib.set_plan(cluster_k=1, workspace_k=split_k // 2)
    try:
        plan = lib.get_plan(M, N, K, split_k)
        if split_k > 1:
            assert plan["workspace_k"] > 1, "this case is meant to exercise the scratch"
        want = torch.full((N, M), float("nan"), dtype=torch.float16, device="cuda")
        ws = torch.empty((split_k, N, M), dtype=torch.float16, device="cuda")
        lib.SpMM_SplitK_API(stream, None, comp_d.data_ptr(), offs_d.data_ptr(), B_d.data_ptr(), want.data_ptr(), M, N, K,
                            ws.data_ptr(), split_k)
        torch.cuda.synchronize()
        # Output buffers are made before the measurement, so that nothing torch does falls between the two readings
        # of the driver's free-memory figure (cudaMemGetInfo), which also sees allocations made inside the library.
        outs = [torch.full((N, M), float("nan"), dtype=torch.float16, device="cuda") for _ in range(3)]
        lib.spmm_splitk_no_alloc(stream, comp_d.data_ptr(), offs_d.data_ptr(), B_d.data_ptr(), outs[2].data_ptr(), M, N,
                                 K, split_k)  # warm-up: the per-device set-up of the first call is behind us
        torch.cuda.synchronize()
        free_before = torch.cuda.mem_get_info()[0]
        for call in range(2):  # the second call finds the first call's partial sums in the scratch
            lib.spmm_splitk_no_alloc(stream, comp_d.data_ptr(), offs_d.data_ptr(), B_d.data_ptr(), outs[call].data_ptr(),
                                     M, N, K, split_k)
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info()[0] == free_before, "device memory was allocated during the calls"
        assert lib.consume_status() == 0
        for call in range(2):
            assert_close(outs[call].cpu().numpy(), want.cpu().numpy().astype(np.float32), f"no-alloc call {call}")
            assert_close(outs[call].cpu().numpy(), oracle.gemm_f32(A, B), f"no-alloc call {call} vs host GEMM")
    finally:
        lib.set_plan()


def test_no_alloc_entry_refuses_oversized_requests(lib, capfd):
    L = lib.library()
    fake = 0x1000  # never dereferenced: the size check comes first
    # 8 * 36864 * 16 * 2 bytes = 9.4 MB > 8 MiB
    assert L.FlashLLM_SpMM_SplitK_NoAlloc(None, fake, fake, fake, fake, 36864, 16, 9216, 8) == 1
    assert "exceeds the built-in" in capfd.readouterr().err
    # without a K split the scratch is not used, so no size is too large for it: this request passes the size check and
    # is turned down only later, for its null buffers
    assert L.FlashLLM_SpMM_SplitK_NoAlloc(None, None, None, None, None, 36864, 128, 9216, 1) == 1
    assert "exceeds the built-in" not in capfd.readouterr().err
