"""The device tiled-CSL encoder must reproduce the host encoder (and so the reference) bit for bit."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _encode_on_device(lib, A_np: np.ndarray, reorder: bool):
    M, K = A_np.shape
    T = (M // 128) * (K // 64)
    A_d = torch.from_numpy(np.ascontiguousarray(A_np.view(np.float16))).cuda()
    offs = torch.full((T + 2,), -7, dtype=torch.int32, device="cuda")
    L = lib.library()
    stream = torch.cuda.current_stream().cuda_stream
    assert L.FlashLLM_EncodeOnDevice_TileOffsets(stream, A_d.data_ptr(), M, K, offs.data_ptr()) == 0
    words = int(offs[T + 1].item()) * 4
    comp = torch.full((max(words, 4),), -1, dtype=torch.int32, device="cuda")
    assert L.FlashLLM_EncodeOnDevice_Pack(stream, A_d.data_ptr(), M, K, offs.data_ptr(), comp.data_ptr(),
                                          1 if reorder else 0) == 0
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    return comp.cpu().numpy().view(np.uint32)[:words], offs.cpu().numpy()


@pytest.mark.parametrize("M,K,sparsity", [(128, 64, 0.8), (128, 64, 0.0), (128, 64, 1.0), (256, 192, 0.7),
                                          (384, 128, 0.999), (1024, 1024, 0.9), (4096, 4096, 0.8), (128, 128, 0.5)])
@pytest.mark.parametrize("reorder", [True, False])
def test_device_encoder_bit_exact(lib, M, K, sparsity, reorder):
    A = lib.synthetic.sparse_uniform_matrix(M, K, sparsity, seed=M + K).numpy()
    comp_h, offs_h, _ = (lib.InitSparseMatrixA_API if reorder else lib.InitSparseMatrixA_API_NoReorder)(A)
    comp_d, offs_d = _encode_on_device(lib, A, reorder)
    assert np.array_equal(offs_d, offs_h)
    assert np.array_equal(comp_d, comp_h)


def test_device_encoder_golden_and_special_values(lib):
    import glob
    import os
    for path in sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz"))):
        g = np.load(path)
        for reorder, key in ((True, "compressed_reorder"), (False, "compressed_noreorder")):
            comp_d, offs_d = _encode_on_device(lib, g["A"], reorder)
            assert np.array_equal(offs_d, g["tile_offsets"]), path
            assert np.array_equal(comp_d, g[key]), (path, reorder)


def test_device_encoded_buffers_feed_the_kernel(lib, oracle):
    from helpers import assert_close
    M, K, N = 1024, 2048, 16
    A = lib.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=9)
    B = lib.synthetic.dense_uniform_matrix(N, K, 10)
    A_d, B_d = A.cuda(), B.cuda()
    T = (M // 128) * (K // 64)
    stream = torch.cuda.current_stream().cuda_stream
    comp, offs, n, words = lib.encode_on_device(
        stream, A_d.data_ptr(), M, K,
        lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device="cuda")),
        lambda n: (lambda t: (t, t.data_ptr()))(torch.empty(n, dtype=torch.int32, device="cuda")),
        lambda owner, i: owner[i].item())
    assert n == T + 2
    C = torch.empty((N, M), dtype=torch.float16, device="cuda")
    lib.SpMM_SplitK_API(stream, None, comp.data_ptr(), offs.data_ptr(), B_d.data_ptr(), C.data_ptr(), M, N, K, None, 1)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    assert_close(C.cpu().numpy(), oracle.gemm_f32(A.numpy(), B.numpy()), "device-encoded SpMM")
