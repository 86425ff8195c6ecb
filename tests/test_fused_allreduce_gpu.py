"""The row-parallel SpMM with the all-reduce fused in (FlashLLM_SpMM_SplitK_AllReduce), with the ranks of the group
emulated on one device: every "rank" has a communicator and a receive buffer on this GPU.  The first kernel of the
fused call (SpMM + stores into every rank's buffer) never waits for anybody, so all ranks' first phases are enqueued
first and their summing phases afterwards, on one stream: no kernel ever waits for a kernel that has not run yet.
The reference does this step with a cuBLAS/SpMM GEMM followed by FasterTransformer's NCCL all-reduce
(third_party/ft.patch:2822-2846 and the out-proj / FFN2 call sites, :1328-1340, :615-633)."""
import numpy as np
import pytest
import torch

from helpers import assert_close, random_problem

pytestmark = pytest.mark.gpu


def _shards(lib, M, K_full, N, world, seed):
    A, B = random_problem(lib, M, K_full, N, 0.8, seed)
    k = K_full // world
    dev = torch.device("cuda:0")
    parts = []
    for r in range(world):
        A_r = np.ascontiguousarray(A[:, r * k:(r + 1) * k])
        B_r = np.ascontiguousarray(B[:, r * k:(r + 1) * k])
        comp, offs, _ = lib.InitSparseMatrixA_API(A_r)
        words = comp.view(np.int32) if comp.size else np.zeros(4, np.int32)
        parts.append((torch.from_numpy(np.ascontiguousarray(words)).to(dev), torch.from_numpy(offs).to(dev),
                      torch.from_numpy(B_r).to(dev)))
    return A, B, parts, k


@pytest.mark.parametrize("M,K_full,N,world", [(1024, 4096, 16, 4), (512, 8192, 8, 8), (256, 1024, 64, 2),
                                              (9216, 9216, 16, 8)])
def test_fused_allreduce_matches_the_unsharded_product(lib, oracle, M, K_full, N, world):
    from flash_llm_b200 import tp_chain
    A, B, parts, k = _shards(lib, M, K_full, N, world, seed=900 + world)
    want = oracle.gemm_f32(A, B)
    stream = torch.cuda.current_stream().cuda_stream
    group = tp_chain.LocalGroup(lib, world, M * N)
    try:
        for call in range(3):  # successive calls alternate between the two halves of the receive buffers
            outs = [torch.full((N, M), float("nan"), dtype=torch.float16, device="cuda") for _ in range(world)]
            for phase in (1, 2):
                for r, (comp, offs, B_r) in enumerate(parts):
                    lib.spmm_splitk_allreduce(group.comms[r], stream, comp.data_ptr(), offs.data_ptr(), B_r.data_ptr(),
                                              outs[r].data_ptr(), M, N, k, phases=phase)
            torch.cuda.synchronize()
            assert lib.consume_status() == 0
            first = outs[0].cpu().numpy()
            assert_close(first, want, f"call {call}")
            for r in range(1, world):  # summed in rank order everywhere: every rank holds the same bits
                assert torch.equal(outs[r], outs[0]), f"rank {r} differs from rank 0 in call {call}"
    finally:
        group.close()


def test_fused_allreduce_adds_the_residual_once(lib, oracle):
    """The decoder layer's residual goes in after the group's sum and before the one rounding, on every rank."""
    from flash_llm_b200 import tp_chain
    M, K_full, N, world = 768, 3072, 16, 4
    A, B, parts, k = _shards(lib, M, K_full, N, world, seed=91)
    bias = lib.synthetic.dense_uniform_matrix(1, M, 92).reshape(M)
    residual = lib.synthetic.dense_uniform_matrix(N, M, 93)
    want = oracle.gemm_f32(A, B) + bias.numpy().astype(np.float32)[None, :] + residual.numpy().astype(np.float32)
    stream = torch.cuda.current_stream().cuda_stream
    group = tp_chain.LocalGroup(lib, world, M * N)
    bias_d, residual_d = bias.cuda(), residual.cuda()
    try:
        outs = [torch.empty((N, M), dtype=torch.float16, device="cuda") for _ in range(world)]
        for phase in (1, 2):
            for r, (comp, offs, B_r) in enumerate(parts):
                lib.spmm_splitk_allreduce(group.comms[r], stream, comp.data_ptr(), offs.data_ptr(), B_r.data_ptr(),
                                          outs[r].data_ptr(), M, N, k, bias=bias_d.data_ptr(),
                                          residual=residual_d.data_ptr(), phases=phase)
        torch.cuda.synchronize()
        assert lib.consume_status() == 0
        assert_close(outs[0].cpu().numpy(), want, "bias + residual on the summed product")
        for r in range(1, world):
            assert torch.equal(outs[r], outs[0])
    finally:
        group.close()


def test_fused_allreduce_applies_bias_and_relu_after_the_sum(lib, oracle):
    from flash_llm_b200 import tp_chain
    M, K_full, N, world = 512, 2048, 16, 2
    A, B, parts, k = _shards(lib, M, K_full, N, world, seed=77)
    bias = lib.synthetic.dense_uniform_matrix(1, M, 78).reshape(M)
    want = np.maximum(oracle.gemm_f32(A, B) + bias.numpy().astype(np.float32)[None, :], 0.0)
    stream = torch.cuda.current_stream().cuda_stream
    group = tp_chain.LocalGroup(lib, world, M * N)
    bias_d = bias.cuda()
    try:
        outs = [torch.empty((N, M), dtype=torch.float16, device="cuda") for _ in range(world)]
        for phase in (1, 2):
            for r, (comp, offs, B_r) in enumerate(parts):
                lib.spmm_splitk_allreduce(group.comms[r], stream, comp.data_ptr(), offs.data_ptr(), B_r.data_ptr(),
                                          outs[r].data_ptr(), M, N, k, bias=bias_d.data_ptr(), activation=lib.ACT_RELU,
                                          phases=phase)
        torch.cuda.synchronize()
        assert lib.consume_status() == 0
        assert_close(outs[1].cpu().numpy(), want, "bias + ReLU on the summed product")
    finally:
        group.close()


def test_missing_peer_is_reported_not_waited_for(lib):
    """A rank whose partner never delivers: the summing kernel's wait is bounded (set to 200 ms here), it then sets status bit 32,
    stores nothing and returns; the context stays usable.  The missing delivery is made on the host (the partner's call
    is simply not issued); nothing on the device faults or spins without a limit."""
    from flash_llm_b200 import tp_chain
    M, K_full, N, world = 256, 1024, 16, 2
    _, _, parts, k = _shards(lib, M, K_full, N, world, seed=5)
    stream = torch.cuda.current_stream().cuda_stream
    group = tp_chain.LocalGroup(lib, world, M * N)
    lib.comm_set_wait_limit(group.comms[0], 200)
    try:
        out = torch.full((N, M), 7.0, dtype=torch.float16, device="cuda")
        comp, offs, B_r = parts[0]
        lib.spmm_splitk_allreduce(group.comms[0], stream, comp.data_ptr(), offs.data_ptr(), B_r.data_ptr(),
                                  out.data_ptr(), M, N, k)  # rank 1 never calls
        torch.cuda.synchronize()
        assert lib.consume_status() & 32
        assert bool((out == 7.0).all()), "the output must be left alone when a partner is missing"
        # the same group cannot be resynchronised (rank 1 is a call behind), but the library itself is fine:
        C = torch.empty((N, M), dtype=torch.float16, device="cuda")
        lib.SpMM_SplitK_API(stream, None, comp.data_ptr(), offs.data_ptr(), B_r.data_ptr(), C.data_ptr(), M, N, k, None, 1)
        torch.cuda.synchronize()
        assert lib.consume_status() == 0
    finally:
        group.close()


def test_fused_allreduce_argument_checks(lib):
    from flash_llm_b200 import tp_chain
    L = lib.library()
    fake = 0x1000
    assert L.FlashLLM_SpMM_SplitK_AllReduce(None, None, fake, fake, fake, fake, 256, 16, 256, None, 0, None, 3) == 1  # no comm
    group = tp_chain.LocalGroup(lib, 2, 256 * 16)
    try:
        # output larger than the communicator was sized for
        assert L.FlashLLM_SpMM_SplitK_AllReduce(group.comms[0], None, fake, fake, fake, fake, 512, 16, 256, None, 0, None, 3) == 1
        assert L.FlashLLM_SpMM_SplitK_AllReduce(group.comms[0], None, fake, fake, fake, fake, 256, 16, 256, None, 0, None, 4) == 1
    finally:
        group.close()
