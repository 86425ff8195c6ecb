"""TEST INFRASTRUCTURE — ctypes front-end of the CPU oracle (``liboracle.so``) and of the
reference library built from its own sources (``_ref/libSpMM_API_ref.so``).

Only the test-suite, the smoke test and the benchmark's CPU-baseline leg import this module;
the shipped package never does.  All arrays are numpy; fp16 data travels as ``uint16`` bit
patterns so that nothing is re-rounded on the way.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
ORACLE_SO = os.path.join(_HERE, "liboracle.so")
REFERENCE_SO = os.path.join(_HERE, "_ref", "libSpMM_API_ref.so")

_u16p = C.POINTER(C.c_uint16)
_u32p = C.POINTER(C.c_uint32)
_i32p = C.POINTER(C.c_int)
_f32p = C.POINTER(C.c_float)


def build(reference: bool = True) -> None:
    """Compile the oracle (and, where the reference tree is present, the reference library)."""
    target = "all" if reference else os.path.join(_HERE, "liboracle.so")
    subprocess.run(["make", "-s", "-f", os.path.join(_HERE, "Makefile"), target], check=True)


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        if not os.path.exists(ORACLE_SO):
            build(reference=False)
        L = C.CDLL(ORACLE_SO)
        for name in ("oracle_encode_reorder", "oracle_encode_noreorder"):
            f = getattr(L, name)
            f.restype = C.c_int
            f.argtypes = [_u16p, C.c_int, C.c_int, C.POINTER(_u32p), C.POINTER(_i32p)]
        L.oracle_free.argtypes = [C.c_void_p]
        L.oracle_decode.argtypes = [_u32p, _i32p, C.c_int, C.c_int, _u16p]
        for name in ("oracle_gemm_f32", "oracle_gemm_f32_timed"):
            getattr(L, name).argtypes = [_u16p, _u16p, _f32p] + [C.c_int] * 5
        L.oracle_spmm_splitk.restype = C.c_int
        L.oracle_spmm_splitk.argtypes = [_u32p, _i32p, _u16p, _u16p] + [C.c_int] * 4
        L.oracle_total_error.restype = C.c_double
        L.oracle_total_error.argtypes = [_u16p, _u16p, C.c_longlong]
        L.oracle_half_to_float.restype = C.c_float
        L.oracle_half_to_float.argtypes = [C.c_uint16]
        L.oracle_float_to_half.restype = C.c_uint16
        L.oracle_float_to_half.argtypes = [C.c_float]
        _lib = L
    return _lib


def _as_u16(a: np.ndarray) -> np.ndarray:
    if a.dtype == np.float16:
        a = a.view(np.uint16)
    assert a.dtype == np.uint16, a.dtype
    return np.ascontiguousarray(a)


def _take(comp_p, offs_p, num_offsets: int, free) -> tuple[np.ndarray, np.ndarray]:
    offs = np.ctypeslib.as_array(offs_p, shape=(num_offsets,)).copy()
    nwords = int(offs[-1]) * 4
    comp = (np.ctypeslib.as_array(comp_p, shape=(max(nwords, 1),))[:nwords]).copy()
    free(comp_p)
    free(offs_p)
    return comp, offs


def encode(A: np.ndarray, reorder: bool = True) -> tuple[np.ndarray, np.ndarray]:
    """Dense [M][K] fp16 -> (Compressed_A uint32[4*TileOffsets[-1]], TileOffsets int32[T+2])."""
    A = _as_u16(A)
    M, K = A.shape
    comp_p, offs_p = _u32p(), _i32p()
    fn = lib().oracle_encode_reorder if reorder else lib().oracle_encode_noreorder
    n = fn(A.ctypes.data_as(_u16p), M, K, C.byref(comp_p), C.byref(offs_p))
    if n < 0:
        raise ValueError(f"M={M} must be a multiple of 128 and K={K} of 64")
    return _take(comp_p, offs_p, n, lambda p: lib().oracle_free(C.cast(p, C.c_void_p)))


def decode(comp: np.ndarray, offs: np.ndarray, M: int, K: int) -> np.ndarray:
    """(Compressed_A, TileOffsets) -> dense [M][K] fp16 bit patterns (uint16)."""
    comp = np.ascontiguousarray(comp, dtype=np.uint32)
    if comp.size == 0:
        comp = np.zeros(1, np.uint32)
    offs = np.ascontiguousarray(offs, dtype=np.int32)
    out = np.empty((M, K), np.uint16)
    lib().oracle_decode(comp.ctypes.data_as(_u32p), offs.ctypes.data_as(_i32p), M, K, out.ctypes.data_as(_u16p))
    return out


def set_threads(n: int) -> None:
    """Host threads used by the OpenMP loops of the oracle (overrides an OMP_NUM_THREADS pinned by a launcher)."""
    lib().oracle_set_threads(int(n))


def gemm_f32(A: np.ndarray, B: np.ndarray, rows: tuple[int, int] | None = None, timed: bool = False) -> np.ndarray:
    """C[N][M] float32 = B[N][K] @ A[M][K]^T on the host; ``rows`` limits the computed A rows."""
    A, B = _as_u16(A), _as_u16(B)
    M, K = A.shape
    N = B.shape[0]
    assert B.shape[1] == K
    out = np.zeros((N, M), np.float32)
    lo, hi = rows if rows is not None else (0, M)
    fn = lib().oracle_gemm_f32_timed if timed else lib().oracle_gemm_f32
    fn(A.ctypes.data_as(_u16p), B.ctypes.data_as(_u16p), out.ctypes.data_as(_f32p), M, N, K, lo, hi)
    return out


def spmm_splitk(comp: np.ndarray, offs: np.ndarray, B: np.ndarray, M: int, N: int, K: int, split_k: int) -> np.ndarray:
    """CPU model of SpMM_SplitK_API with the reference's split-K rounding; returns C[N][M] float16."""
    comp = np.ascontiguousarray(comp, dtype=np.uint32)
    if comp.size == 0:
        comp = np.zeros(1, np.uint32)
    offs = np.ascontiguousarray(offs, dtype=np.int32)
    B = _as_u16(B)
    out = np.zeros((N, M), np.uint16)
    rc = lib().oracle_spmm_splitk(comp.ctypes.data_as(_u32p), offs.ctypes.data_as(_i32p), B.ctypes.data_as(_u16p),
                                  out.ctypes.data_as(_u16p), M, N, K, split_k)
    if rc != 0:
        raise ValueError(f"Split_K={split_k} leaves an empty K batch for K={K}")
    return out.view(np.float16)


def total_error(ref: np.ndarray, other: np.ndarray) -> float:
    ref, other = _as_u16(ref), _as_u16(other)
    return float(lib().oracle_total_error(ref.ctypes.data_as(_u16p), other.ctypes.data_as(_u16p), ref.size))


# ----------------------------------------------------------------------------- reference library

# C++-mangled exports of the reference (build/SpMM_API.cuh:38-58)
MANGLED = {
    "SpMM_SplitK_API": "_Z15SpMM_SplitK_APIP11CUstream_stPK6__halfPK5uint4PKiS3_PS1_iiiS9_i",
    "InitSparseMatrixA_API": "_Z21InitSparseMatrixA_APIP6__halfiiiPPjPPi",
    "InitSparseMatrixA_API_NoReorder": "_Z31InitSparseMatrixA_API_NoReorderP6__halfiiiPPjPPi",
}

_ref = None


def reference_available() -> bool:
    return os.path.exists(REFERENCE_SO)


def reference_lib() -> C.CDLL:
    """The unmodified reference, compiled from its own sources for sm_100a (host encoder runs anywhere)."""
    global _ref
    if _ref is None:
        L = C.CDLL(REFERENCE_SO)
        for key in ("InitSparseMatrixA_API", "InitSparseMatrixA_API_NoReorder"):
            f = getattr(L, MANGLED[key])
            f.restype = C.c_int
            f.argtypes = [_u16p, C.c_int, C.c_int, C.c_int, C.POINTER(_u32p), C.POINTER(_i32p)]
        f = getattr(L, MANGLED["SpMM_SplitK_API"])
        f.restype = C.c_int
        f.argtypes = [C.c_void_p] * 6 + [C.c_int] * 3 + [C.c_void_p, C.c_int]
        _ref = L
    return _ref


def reference_encode(A: np.ndarray, reorder: bool = True) -> tuple[np.ndarray, np.ndarray]:
    A = _as_u16(A)
    M, K = A.shape
    L = reference_lib()
    fn = getattr(L, MANGLED["InitSparseMatrixA_API" if reorder else "InitSparseMatrixA_API_NoReorder"])
    comp_p, offs_p = _u32p(), _i32p()
    n = fn(A.ctypes.data_as(_u16p), M, 0, K, C.byref(comp_p), C.byref(offs_p))
    libc = C.CDLL(None)
    libc.free.argtypes = [C.c_void_p]
    return _take(comp_p, offs_p, n, lambda p: libc.free(C.cast(p, C.c_void_p)))


def reference_spmm(stream: int, comp_dev: int, offs_dev: int, B_dev: int, C_dev: int, M: int, N: int, K: int,
                   workspace_dev: int, split_k: int) -> int:
    """Launches the reference kernel (device pointers as integers); returns its cudaError_t."""
    fn = getattr(reference_lib(), MANGLED["SpMM_SplitK_API"])
    return fn(stream, None, comp_dev, offs_dev, B_dev, C_dev, M, N, K, workspace_dev, split_k)
