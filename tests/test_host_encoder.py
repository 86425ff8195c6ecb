"""Host side of the product on CPU: the tiled-CSL encoders of libSpMM_API.so against the oracle and the golden
fixtures, the exported symbol list, argument checks that return before any CUDA call, and the file converter."""
import ctypes as C
import glob
import os
import re

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_library_encoders_match_golden(lib, path):
    g = np.load(path)
    comp, offs, n = lib.InitSparseMatrixA_API(g["A"])
    assert n == offs.size == g["tile_offsets"].size
    assert np.array_equal(offs, g["tile_offsets"]) and np.array_equal(comp, g["compressed_reorder"])
    comp, offs, n = lib.InitSparseMatrixA_API_NoReorder(g["A"])
    assert np.array_equal(offs, g["tile_offsets"]) and np.array_equal(comp, g["compressed_noreorder"])


@pytest.mark.parametrize("M,K,sparsity", [(128, 64, 0.8), (384, 448, 0.7), (1024, 1024, 0.9), (2048, 512, 0.8),
                                          (128, 4096, 0.95), (256, 128, 0.0), (256, 128, 1.0)])
def test_library_encoders_match_oracle(lib, oracle, M, K, sparsity):
    A = lib.synthetic.sparse_uniform_matrix(M, K, sparsity, seed=M * 31 + K).numpy()
    for reorder, fn in ((True, lib.InitSparseMatrixA_API), (False, lib.InitSparseMatrixA_API_NoReorder)):
        comp, offs, n = fn(A)
        comp_o, offs_o = oracle.encode(A, reorder)
        assert n == (M // 128) * (K // 64) + 2
        assert np.array_equal(offs, offs_o) and np.array_equal(comp, comp_o)


def test_format_invariants(lib, oracle):
    M, K = 512, 256
    A = lib.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=99).numpy()
    comp, offs, n = lib.InitSparseMatrixA_API(A)
    T = (M // 128) * (K // 64)
    assert offs[0] == 0 and offs[T + 1] == offs[T] and np.all(np.diff(offs) >= 0)
    assert comp.size == 4 * offs[T]
    assert np.all((comp >> 16) < 8192)
    assert np.array_equal(oracle.decode(comp, offs, M, K), A.view(np.uint16))
    # per tile: at most three padding words, each +0.0 aimed at a zero cell
    Ab = A.view(np.uint16)
    for t in range(T):
        words = comp[4 * offs[t]:4 * offs[t + 1]]
        i, j = divmod(t, K // 64)
        tile = Ab[i * 128:(i + 1) * 128, j * 64:(j + 1) * 64]
        pads = words[(words & 0xFFFF) == 0]
        assert pads.size == words.size - np.count_nonzero(tile) and pads.size <= 3
        for w in pads:
            loc = int(w >> 16)
            r, c = loc >> 6, (loc & 63) ^ (((loc >> 6) & 7) << 3)
            assert tile[r, c] == 0


def test_row_shards_encode_independently(lib):
    """Row (output-feature) sharding needs no exchange: a shard's encoding is a slice of the full one."""
    M, K, world = 1024, 256, 4
    A = lib.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=5).numpy()
    comp, offs, _ = lib.InitSparseMatrixA_API(A)
    kt = K // 64
    for rank in range(world):
        rows = slice(rank * M // world, (rank + 1) * M // world)
        c, o, _ = lib.InitSparseMatrixA_API(A[rows])
        t0 = (rows.start // 128) * kt
        t1 = (rows.stop // 128) * kt
        assert np.array_equal(o[:-1], offs[t0:t1 + 1] - offs[t0])
        assert np.array_equal(c, comp[4 * offs[t0]:4 * offs[t1]])


def test_bad_shapes_rejected(lib):
    with pytest.raises(lib.FlashLLMError):
        lib.InitSparseMatrixA_API(np.zeros((100, 64), np.float16))
    with pytest.raises(lib.FlashLLMError):
        lib.InitSparseMatrixA_API(np.zeros((128, 65), np.float16))


def test_every_declared_symbol_is_exported(lib):
    text = open(os.path.join(ROOT, "include", "SpMM_API.cuh")).read()
    c_block = text[text.index('extern "C" {'):]
    names = set(re.findall(r"\b(FlashLLM_\w+|GenSparseMatrixBinFile)\s*\(", c_block))
    assert len(names) >= 12
    L = lib.library()
    for name in sorted(names):
        assert getattr(L, name) is not None, name
    # reference-compatible C++ symbols (Itanium mangling of the signatures in the reference header)
    for mangled in ("_Z15SpMM_SplitK_APIP11CUstream_stPK6__halfPK5uint4PKiS3_PS1_iiiS9_i",
                    "_Z21InitSparseMatrixA_APIP6__halfiiiPPjPPi",
                    "_Z31InitSparseMatrixA_API_NoReorderP6__halfiiiPPjPPi"):
        assert getattr(L, mangled) is not None, mangled


def test_spmm_argument_checks_without_gpu(lib, capfd):
    """Checks that run before any CUDA call: unsupported N prints the reference's message and returns
    cudaErrorUnknown (999); bad shapes and null pointers return cudaErrorInvalidValue (1)."""
    L = lib.library()
    fake = 0x1000  # never dereferenced: every call below is rejected first
    assert L.FlashLLM_SpMM_SplitK(None, None, fake, fake, fake, fake, 256, 24, 64, None, 1) == 999
    assert "Unsupported N dimension 24" in capfd.readouterr().out
    assert L.FlashLLM_SpMM_SplitK(None, None, fake, fake, fake, fake, 100, 16, 64, None, 1) == 1
    assert L.FlashLLM_SpMM_SplitK(None, None, fake, fake, fake, fake, 128, 16, 96, None, 1) == 1
    assert L.FlashLLM_SpMM_SplitK(None, None, None, fake, fake, fake, 128, 16, 64, None, 1) == 1
    assert L.FlashLLM_SpMM_SplitK(None, None, fake + 4, fake, fake, fake, 128, 16, 64, None, 1) == 1
    assert L.FlashLLM_SpMM_SplitK(None, None, fake, fake, fake, fake, 128, 16, 64, None, 0) == 1
    assert L.FlashLLM_SpMM_SplitK(None, None, fake, fake, fake, fake, 128, 16, 64, None, 2) == 1  # no workspace
    assert L.FlashLLM_SplitK_Reduction(None, fake, fake, 10, 3, 2) == 1  # M*N not a multiple of 8
    assert L.FlashLLM_EncodeOnDevice_TileOffsets(None, fake, 100, 64, fake) == 1


def test_gen_sparse_matrix_bin_file(lib, oracle, tmp_path):
    M, K = 256, 128
    A = lib.synthetic.sparse_uniform_matrix(M, K, 0.8, seed=3).numpy()
    dense = tmp_path / "w.bin"
    A.tofile(dense)
    out = [str(tmp_path / n) for n in ("w.NZWeights.bin", "w.TileOffsets.bin", "w.OutputSizes.bin")]
    lib.GenSparseMatrixBinFile(str(dense), M, K, *out)
    comp_o, offs_o = oracle.encode(A, True)
    sizes = np.fromfile(out[2], np.int32)
    assert sizes.tolist() == [comp_o.size, offs_o.size]
    assert np.array_equal(np.fromfile(out[0], np.uint32), comp_o)
    assert np.array_equal(np.fromfile(out[1], np.int32), offs_o)
