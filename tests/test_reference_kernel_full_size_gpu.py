"""This library against the reference's own SpMM kernel at the full sizes of the benchmark configurations.

The reference (csrc/SpMM_API.cu:55-130 and the kernels behind it) is compiled unmodified for sm_100a into
oracle/_ref/ by oracle/Makefile; both kernels run on the same device buffers (same tiled-CSL encoding, same B) and
the whole outputs are compared on the device.  Split_K is the reference's own table (kernel_benchmark/benchmark.sh:
13-15) unless a configuration names one.  Shapes the reference kernel cannot run (M not a multiple of 256 at
N <= 32) are covered against the host GEMM in test_full_size_gpu.py instead."""
import pytest
import torch

from helpers import assert_close_device
from oracle import cpu_oracle

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(not cpu_oracle.reference_available(), reason="oracle/_ref has not been built")]

# Split_K per (M, K) as the reference benchmark tunes it (kernel_benchmark/benchmark.sh:13-15)
REFERENCE_SPLIT_K = {(27648, 9216): 2, (9216, 9216): 6, (36864, 9216): 3, (9216, 36864): 6,
                     (36864, 12288): 3, (12288, 12288): 9, (49152, 12288): 9, (12288, 49152): 9}


def _encode(lib, M, K, sparsity, seed, rows=None):
    """Seeded A (optionally the row range `rows` of it) encoded on the device; the dense matrix is dropped."""
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    A = lib.synthetic.sparse_uniform_matrix(M, K, sparsity, seed, device=dev)
    if rows is not None:
        A = A[rows[0]:rows[1]].contiguous()
    # a few spare elements behind each buffer: the reference kernel's last CTA reads one int past TileOffsets[T+1]
    # (csrc/SpMM_Kernel.cuh:309-315)
    mk = lambda n: (lambda t: (t, t.data_ptr()))(torch.zeros(n + 64, dtype=torch.int32, device=dev))  # noqa: E731
    comp, offs, _, _ = lib.encode_on_device(stream, A.data_ptr(), A.shape[0], K, mk, mk, lambda o, i: o[i].item())
    return comp, offs


def _both(lib, comp, offs, M, K, N, split_k, seed, what):
    dev = torch.device("cuda:0")
    stream = torch.cuda.current_stream().cuda_stream
    B = lib.synthetic.dense_uniform_matrix(N, K, seed ^ 0xB, device=dev)
    ws = torch.empty((split_k, N, M), dtype=torch.float16, device=dev)
    mine = torch.full((N, M), float("nan"), dtype=torch.float16, device=dev)
    theirs = torch.full((N, M), float("nan"), dtype=torch.float16, device=dev)
    lib.SpMM_SplitK_API(stream, None, comp.data_ptr(), offs.data_ptr(), B.data_ptr(), mine.data_ptr(), M, N, K,
                        ws.data_ptr(), split_k)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    rc = cpu_oracle.reference_spmm(stream, comp.data_ptr(), offs.data_ptr(), B.data_ptr(), theirs.data_ptr(), M, N, K,
                                   ws.data_ptr(), split_k)
    torch.cuda.synchronize()
    assert rc == 0
    assert_close_device(mine, theirs, what, fp16_partials=split_k if split_k > 1 else 0)


@pytest.mark.parametrize("sparsity", [0.7, 0.8, 0.9])
@pytest.mark.parametrize("M,K", [(27648, 9216), (9216, 9216), (36864, 9216), (9216, 36864)])
def test_opt66b_shapes_whole_output(lib, M, K, sparsity):
    comp, offs = _encode(lib, M, K, sparsity, seed=M + K)
    for N in (8, 16, 32):
        _both(lib, comp, offs, M, K, N, REFERENCE_SPLIT_K[(M, K)], M + K + N, f"{M}x{K} N={N} s={sparsity}")


@pytest.mark.parametrize("M,K", [(36864, 12288), (12288, 12288), (49152, 12288), (12288, 49152)])
def test_opt175b_shapes_whole_output(lib, M, K):
    comp, offs = _encode(lib, M, K, 0.8, seed=M + K)
    for N in (8, 16, 32, 64):
        _both(lib, comp, offs, M, K, N, REFERENCE_SPLIT_K[(M, K)], M + K + N, f"{M}x{K} N={N}")


@pytest.mark.parametrize("shards", [2, 4, 8])
@pytest.mark.parametrize("M,K", [(36864, 12288), (12288, 12288), (49152, 12288), (12288, 49152)])
def test_opt175b_row_shards_whole_output(lib, M, K, shards):
    rows = M // shards
    for rank in sorted({0, shards - 1}):
        comp, offs = _encode(lib, M, K, 0.8, seed=M + K, rows=(rank * rows, (rank + 1) * rows))
        _both(lib, comp, offs, rows, K, 16, REFERENCE_SPLIT_K[(M, K)], M + K + rank,
              f"rows {rank}/{shards} of {M}x{K}")


@pytest.mark.parametrize("split_k", [1, 2, 4, 8])
def test_split_k_stress_whole_output(lib, split_k):
    M, K, N = 12288, 49152, 8
    comp, offs = _encode(lib, M, K, 0.9, seed=4)
    _both(lib, comp, offs, M, K, N, split_k, 40 + split_k, f"{M}x{K} N={N} Split_K={split_k}")


@pytest.mark.parametrize("split_k", [1, 4, 8])
def test_small_m_long_k_whole_output(lib, split_k):
    M, K, N = 2048, 32768, 16
    comp, offs = _encode(lib, M, K, 0.7, seed=5)
    _both(lib, comp, offs, M, K, N, split_k, 50 + split_k, f"{M}x{K} N={N} Split_K={split_k}")
