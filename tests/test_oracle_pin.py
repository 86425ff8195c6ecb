"""Pins the CPU oracle: against the golden fixtures made from the unmodified reference encoder (always),
and against that encoder itself on fresh random matrices where its build is present."""
import glob
import os

import numpy as np
import pytest

GOLDEN = sorted(glob.glob(os.path.join(os.path.dirname(__file__), "golden", "*.npz")))


def test_golden_fixtures_exist():
    assert len(GOLDEN) >= 8


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_matches_golden(oracle, path):
    g = np.load(path)
    for reorder, key in ((True, "compressed_reorder"), (False, "compressed_noreorder")):
        comp, offs = oracle.encode(g["A"], reorder)
        assert np.array_equal(offs, g["tile_offsets"])
        assert np.array_equal(comp, g[key])


@pytest.mark.parametrize("path", GOLDEN, ids=[os.path.basename(p)[:-4] for p in GOLDEN])
def test_oracle_decode_of_golden(oracle, path):
    g = np.load(path)
    A = g["A"]
    M, K = A.shape
    kept = ((A & 0x7FFF) != 0) & ((A & 0x7FFF) <= 0x7C00)
    dec = oracle.decode(g["compressed_reorder"], g["tile_offsets"], M, K)
    assert np.array_equal(dec[kept], A[kept])
    assert np.all(dec[~kept] == 0)
    # scan-order padding keeps the bits of the first zero-testing cells (-0.0 or NaN may reappear there)
    dec2 = oracle.decode(g["compressed_noreorder"], g["tile_offsets"], M, K)
    assert np.array_equal(dec2[kept], A[kept])
    leftovers = dec2[~kept]
    assert np.all((leftovers == 0) | (leftovers == A[~kept]))


@pytest.mark.parametrize("M,K,sparsity,seed", [(128, 64, 0.8, 1), (256, 256, 0.6, 2), (512, 192, 0.93, 3),
                                               (128, 320, 0.3, 4), (1024, 512, 0.8, 5)])
def test_oracle_matches_reference_encoder(oracle, M, K, sparsity, seed):
    if not oracle.reference_available():
        pytest.skip("reference build (oracle/_ref) not present")
    rng = np.random.default_rng(seed)
    A = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    A[rng.random((M, K)) < sparsity] = 0
    for reorder in (True, False):
        comp, offs = oracle.encode(A, reorder)
        comp_ref, offs_ref = oracle.reference_encode(A, reorder)
        assert np.array_equal(offs, offs_ref)
        assert np.array_equal(comp, comp_ref)


def test_half_conversions_match_numpy(oracle):
    L = oracle.lib()
    bits = np.arange(0, 65536, 7, dtype=np.uint16)
    vals = bits.view(np.float16).astype(np.float32)
    for b, v in zip(bits.tolist(), vals.tolist()):
        got = L.oracle_half_to_float(b)
        assert (np.isnan(v) and np.isnan(got)) or got == v
    rng = np.random.default_rng(0)
    xs = (rng.standard_normal(4000) * 10.0 ** rng.integers(-9, 6, 4000)).astype(np.float32)
    xs = np.concatenate([xs, np.array([65504, 65519.9, 65520, 1e9, 2.0 ** -24, 2.0 ** -25, 2.0 ** -25 * 1.0001,
                                       6.1e-5, 0.0, -0.0], np.float32)])
    with np.errstate(over="ignore"):
        want = xs.astype(np.float16).view(np.uint16)
    got = np.array([L.oracle_float_to_half(float(x)) for x in xs], np.uint16)
    assert np.array_equal(got, want)


def test_oracle_spmm_matches_dense_gemm(oracle):
    rng = np.random.default_rng(7)
    M, K, N = 256, 384, 16
    A = rng.uniform(-1, 1, (M, K)).astype(np.float16)
    A[rng.random((M, K)) < 0.8] = 0
    B = rng.uniform(-1, 1, (N, K)).astype(np.float16)
    comp, offs = oracle.encode(A)
    want = B.astype(np.float64) @ A.astype(np.float64).T
    dense = oracle.gemm_f32(A, B)
    assert np.allclose(dense, want, rtol=1e-6, atol=1e-6)
    for split_k in (1, 2, 3, 6):
        got = oracle.spmm_splitk(comp, offs, B, M, N, K, split_k).astype(np.float64)
        assert np.max(np.abs(got - want)) <= 2e-3 * np.max(np.abs(want)) * (1 + split_k)
    with pytest.raises(ValueError):
        oracle.spmm_splitk(comp, offs, B, M, N, K, 5)  # ceil(6/5)=2 -> last batch would start past K
