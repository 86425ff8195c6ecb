"""The PyTorch operators ``torch.ops.flashllm.{encode,spmm,spmm_epilogue}``: registration, shape inference and
refusals on CPU; parity with the CPU oracle on a GPU."""
import numpy as np
import pytest
import torch

from helpers import assert_close, random_problem


@pytest.fixture(scope="module")
def ops(lib):
    from flash_llm_b200 import torch_op  # noqa: F401  (registers the operators)
    return torch.ops.flashllm


def test_operators_are_registered_with_their_schemas(ops):
    assert "int M, int split_k=1" in str(ops.spmm.default._schema)
    assert "Tensor? bias=None, int activation=0, Tensor? residual=None" in str(ops.spmm_epilogue.default._schema)
    assert "-> (Tensor, Tensor)" in str(ops.encode.default._schema)


def test_shape_inference_on_meta_tensors(ops):
    comp = torch.empty(1024, dtype=torch.int32, device="meta")
    offs = torch.empty((256 // 128) * (512 // 64) + 2, dtype=torch.int32, device="meta")
    B = torch.empty((16, 512), dtype=torch.float16, device="meta")
    C = ops.spmm(comp, offs, B, 256, 4)
    assert C.shape == (16, 256) and C.dtype == torch.float16 and C.device.type == "meta"
    C = ops.spmm_epilogue(comp, offs, B, 256, 1, None, 1, torch.empty((16, 256), dtype=torch.float16, device="meta"))
    assert C.shape == (16, 256)


def test_cpu_tensors_are_refused_not_computed(ops):
    comp = torch.zeros(8, dtype=torch.int32)
    offs = torch.zeros(2 * 8 + 2, dtype=torch.int32)
    B = torch.zeros((16, 512), dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.spmm(comp, offs, B, 256)
    with pytest.raises(RuntimeError, match="no CPU implementation"):
        ops.encode(torch.zeros((128, 64), dtype=torch.float16))


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,N,split_k", [(512, 1024, 16, 4), (256, 2048, 64, 1), (384, 768, 128, 2)])
def test_encode_then_spmm_matches_the_oracle(lib, oracle, ops, M, K, N, split_k):
    A, B = random_problem(lib, M, K, N, 0.8, 600 + N)
    A_d, B_d = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    comp, offs = ops.encode(A_d)
    host_comp, host_offs, _ = lib.InitSparseMatrixA_API(A)
    assert np.array_equal(offs.cpu().numpy(), host_offs)
    assert np.array_equal(comp.cpu().numpy().view(np.uint32), host_comp.view(np.uint32).reshape(-1))
    C = ops.spmm(comp, offs, B_d, M, split_k)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    assert_close(C.cpu().numpy(), oracle.gemm_f32(A, B), f"torch op M={M} K={K} N={N}")


@pytest.mark.gpu
def test_epilogue_operator_and_a_side_stream(lib, oracle, ops):
    M, K, N = 512, 1024, 32
    A, B = random_problem(lib, M, K, N, 0.8, 611)
    rng = np.random.default_rng(612)
    bias = (rng.standard_normal(M) * 2).astype(np.float16)
    residual = (rng.standard_normal((N, M)) * 4).astype(np.float16)
    want = np.maximum(oracle.gemm_f32(A, B) + bias.astype(np.float32)[None, :], 0) + residual.astype(np.float32)
    A_d, B_d = torch.from_numpy(A).cuda(), torch.from_numpy(B).cuda()
    bias_d, res_d = torch.from_numpy(bias).cuda(), torch.from_numpy(residual).cuda()
    comp, offs = ops.encode(A_d)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # the operator launches on whatever stream is current
        C = ops.spmm_epilogue(comp, offs, B_d, M, 2, bias_d, lib.ACT_RELU, res_d)
    side.synchronize()
    assert lib.consume_status() == 0
    assert_close(C.cpu().numpy(), want, "torch op with bias, ReLU and residual")


@pytest.mark.gpu
def test_operator_refuses_mismatched_operands(lib, ops):
    A, B = random_problem(lib, 256, 512, 16, 0.8, 620)
    comp, offs = ops.encode(torch.from_numpy(A).cuda())
    B_d = torch.from_numpy(B).cuda()
    with pytest.raises(RuntimeError, match="does not belong"):
        ops.spmm(comp, offs, B_d, 512)
    with pytest.raises(RuntimeError, match="contiguous fp16"):
        ops.spmm(comp, offs, B_d.float(), 256)
    with pytest.raises(RuntimeError, match="bias must be"):
        ops.spmm_epilogue(comp, offs, B_d, 256, 1, torch.zeros(7, dtype=torch.float16, device="cuda"))
