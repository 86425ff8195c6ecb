"""The on-disk form of a converted model: the three files per matrix written by GenSparseMatrixBinFile (reference
csrc/SpMM_API.cu:500-555) and the three per-rank lists written by the reference's converter
(end2end_inference/ft_tools/huggingface_opt_convert_Phase2.py:188-195), read back the way the patched
FasterTransformer loads them (third_party/ft.patch:1863-1965, 3743-3790)."""
import numpy as np
import pytest
import torch


def _convert(lib, tmp_path, M, K, sparsity, seed, name="w"):
    A = lib.synthetic.sparse_uniform_matrix(M, K, sparsity, seed=seed).numpy()
    dense = tmp_path / f"{name}.bin"
    A.tofile(dense)
    out = [str(tmp_path / f"{name}.{part}.bin") for part in ("NZWeights", "TileOffsets", "OutputSizes")]
    lib.GenSparseMatrixBinFile(str(dense), M, K, *out)
    return A, str(dense), out


@pytest.mark.parametrize("M,K,sparsity", [(256, 128, 0.8), (128, 64, 1.0), (384, 256, 0.3)])
def test_reader_round_trip(lib, oracle, tmp_path, M, K, sparsity):
    A, _, (nz, to, sizes) = _convert(lib, tmp_path, M, K, sparsity, seed=5)
    nnz, num_offsets = lib.read_output_sizes(sizes)
    comp, offs = lib.read_sparse_matrix_bin_files(nz, to, nnz, num_offsets)
    comp_o, offs_o = oracle.encode(A, True)
    assert num_offsets == (M // 128) * (K // 64) + 2 and nnz == comp_o.size
    assert np.array_equal(comp, comp_o) and np.array_equal(offs, offs_o)
    assert np.array_equal(oracle.decode(comp, offs, M, K).view(np.uint16) & 0x7FFF, A.view(np.uint16) & 0x7FFF)


def test_reader_rejects_bad_files(lib, tmp_path):
    _, _, (nz, to, sizes) = _convert(lib, tmp_path, 256, 128, 0.8, seed=6)
    nnz, num_offsets = lib.read_output_sizes(sizes)
    with pytest.raises(lib.FlashLLMError, match="cannot be opened"):
        lib.read_output_sizes(str(tmp_path / "missing.bin"))
    with pytest.raises(lib.FlashLLMError, match="shorter"):
        lib.read_sparse_matrix_bin_files(nz, to, nnz, num_offsets + 1)
    with pytest.raises(lib.FlashLLMError, match="well-formed"):  # a word count that disagrees with the offsets
        lib.read_sparse_matrix_bin_files(nz, to, nnz - 4, num_offsets)
    offs = np.fromfile(to, np.int32)
    offs[2] = offs[1] - 1  # offsets that run backwards
    bad = tmp_path / "bad.TileOffsets.bin"
    offs.tofile(bad)
    with pytest.raises(lib.FlashLLMError, match="well-formed"):
        lib.read_sparse_matrix_bin_files(nz, str(bad), nnz, num_offsets)
    np.array([nnz], np.int32).tofile(tmp_path / "short.OutputSizes.bin")
    with pytest.raises(lib.FlashLLMError, match="shorter"):
        lib.read_output_sizes(str(tmp_path / "short.OutputSizes.bin"))


def test_rank_lists_round_trip(lib, tmp_path):
    layers = 3
    nnz = np.arange(1, 4 * layers + 1, dtype=np.int32) * 4
    num_offsets = np.arange(3, 4 * layers + 3, dtype=np.int32)
    split_k = np.tile(np.array([2, 6, 3, 6], np.int32), layers)
    nnz[5] = num_offsets[5] = split_k[5] = 0  # a matrix the converter left dense
    for rank in (0, 1):
        lib.write_rank_lists(str(tmp_path), rank, nnz + 4 * rank * (nnz > 0), num_offsets, split_k)
    # the files are what numpy's tofile of int32 arrays gives, as the reference's converter writes them
    assert np.array_equal(np.fromfile(tmp_path / "SplitK_List.1.bin", np.int32), split_k)
    assert np.array_equal(np.fromfile(tmp_path / "NNZ_List.0.bin", np.int32), nnz)
    for rank in (0, 1):
        a, b, c = lib.read_rank_lists(str(tmp_path), rank, 4 * layers)
        want = nnz + 4 * rank * (nnz > 0)
        assert np.array_equal(a, want) and np.array_equal(b, num_offsets) and np.array_equal(c, split_k)
    with pytest.raises(lib.FlashLLMError, match="shorter"):
        lib.read_rank_lists(str(tmp_path), 0, 4 * layers + 1)
    with pytest.raises(lib.FlashLLMError, match="cannot be opened"):
        lib.read_rank_lists(str(tmp_path), 2, 4 * layers)
    np.array([8, 0], np.int32).tofile(tmp_path / "NNZ_List.3.bin")  # positive NNZ without offsets or Split_K
    np.array([0, 0], np.int32).tofile(tmp_path / "NumOffsets_List.3.bin")
    np.array([0, 0], np.int32).tofile(tmp_path / "SplitK_List.3.bin")
    with pytest.raises(lib.FlashLLMError, match="well-formed"):
        lib.read_rank_lists(str(tmp_path), 3, 2)


@pytest.mark.gpu
@pytest.mark.parametrize("M,K,sparsity", [(512, 1024, 0.8), (128, 64, 1.0), (256, 192, 0.0)])
def test_device_converter_writes_the_same_bytes(lib, tmp_path, M, K, sparsity):
    _, dense, host_out = _convert(lib, tmp_path, M, K, sparsity, seed=8)
    dev_out = [str(tmp_path / f"d.{part}.bin") for part in ("NZWeights", "TileOffsets", "OutputSizes")]
    lib.gen_sparse_matrix_bin_file_device(dense, M, K, *dev_out)
    for h, d in zip(host_out, dev_out):
        assert open(h, "rb").read() == open(d, "rb").read(), d
    assert lib.consume_status() == 0


@pytest.mark.gpu
def test_loader_fills_device_buffers_for_spmm(lib, oracle, tmp_path):
    from helpers import assert_close
    M, K, N = 512, 1024, 16
    A, _, (nz, to, sizes) = _convert(lib, tmp_path, M, K, 0.8, seed=9)
    B = lib.synthetic.dense_uniform_matrix(N, K, seed=10)
    nnz, num_offsets = lib.read_output_sizes(sizes)
    comp_d = torch.empty(nnz, dtype=torch.int32, device="cuda")
    offs_d = torch.empty(num_offsets, dtype=torch.int32, device="cuda")
    lib.load_sparse_matrix_bin_files(nz, to, nnz, num_offsets, comp_d.data_ptr(), offs_d.data_ptr())
    C = torch.empty((N, M), dtype=torch.float16, device="cuda")
    B_d = B.cuda()
    lib.SpMM_SplitK_API(torch.cuda.current_stream().cuda_stream, None, comp_d.data_ptr(), offs_d.data_ptr(),
                        B_d.data_ptr(), C.data_ptr(), M, N, K, None, 1)
    torch.cuda.synchronize()
    assert lib.consume_status() == 0
    assert_close(C.cpu().numpy(), oracle.gemm_f32(A, B.numpy()), "SpMM on loaded files")
