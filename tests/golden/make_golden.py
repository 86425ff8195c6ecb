"""Generates the golden fixtures of this directory from the UNMODIFIED reference encoder.

Run where the reference tree is available (the oracle Makefile compiles it from its own sources into
oracle/_ref/):   python tests/golden/make_golden.py
Each fixture is a small dense fp16 matrix (as uint16 bit patterns) with the reference's
InitSparseMatrixA_API and InitSparseMatrixA_API_NoReorder outputs for it.  The inputs come from numpy's
PCG64 with the seeds below and include the special values the encoder treats specially (+-0, NaN,
subnormals, infinities), empty tiles, fully dense tiles and every padding remainder.
"""
import os
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))

from oracle import cpu_oracle as o  # noqa: E402

CASES = [
    # name, M, K, sparsity, seed, special values
    ("one_tile_80", 128, 64, 0.80, 11, False),
    ("one_tile_dense", 128, 64, 0.0, 12, False),
    ("one_tile_empty", 128, 64, 1.0, 13, False),
    ("two_by_three_70", 256, 192, 0.70, 14, True),
    ("three_by_two_90", 384, 128, 0.90, 15, True),
    ("sparse_999", 256, 128, 0.999, 16, False),
    ("half_dense_50", 128, 128, 0.50, 17, True),
]


def make_matrix(M, K, sparsity, seed, special):
    rng = np.random.default_rng(seed)
    A = rng.uniform(-1.0, 1.0, (M, K)).astype(np.float16)
    A[rng.random((M, K)) < sparsity] = 0
    bits = A.view(np.uint16).copy()
    if special:
        flat = bits.reshape(-1)
        idx = rng.choice(flat.size, 160, replace=False)
        flat[idx[0:40]] = 0x8000    # -0.0: treated as zero
        flat[idx[40:80]] = 0x7E00   # NaN: fails the > 0 test, dropped
        flat[idx[80:120]] = 0x0001  # smallest subnormal: kept
        flat[idx[120:140]] = 0x7C00  # +inf: kept
        flat[idx[140:160]] = 0xFC00  # -inf: kept
    return bits


def main():
    assert o.reference_available(), "build oracle/_ref first (make -C oracle)"
    for name, M, K, sparsity, seed, special in CASES:
        bits = make_matrix(M, K, sparsity, seed, special)
        comp_r, offs_r = o.reference_encode(bits, reorder=True)
        comp_s, offs_s = o.reference_encode(bits, reorder=False)
        assert np.array_equal(offs_r, offs_s)
        np.savez_compressed(os.path.join(HERE, name + ".npz"), A=bits, compressed_reorder=comp_r,
                            compressed_noreorder=comp_s, tile_offsets=offs_r)
        print(name, bits.shape, "words", comp_r.size)
    # remainders 1..3 of the padding rule and a single non-zero in each corner of a tile
    bits = np.zeros((128, 64), np.uint16)
    for r, c in ((0, 0), (0, 63), (127, 0), (127, 63), (64, 31)):
        bits[r, c] = 0x3C00
    comp_r, offs_r = o.reference_encode(bits, True)
    comp_s, _ = o.reference_encode(bits, False)
    np.savez_compressed(os.path.join(HERE, "corners.npz"), A=bits, compressed_reorder=comp_r,
                        compressed_noreorder=comp_s, tile_offsets=offs_r)
    print("corners", comp_r.size)


if __name__ == "__main__":
    main()
