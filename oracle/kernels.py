"""ctypes face of oracle/kernels_oracle.c (test infrastructure; see that file's header)."""
from __future__ import annotations

import ctypes as C
import subprocess
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_SO = _HERE / "liboracle_kernels.so"
_SRC = _HERE / "kernels_oracle.c"


def _build() -> None:
    if not _SO.exists() or _SO.stat().st_mtime < _SRC.stat().st_mtime:
        subprocess.check_call(["/usr/bin/gcc" if Path("/usr/bin/gcc").exists() else "gcc", "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-o", str(_SO), str(_SRC), "-lm"])


_build()
_lib = C.CDLL(str(_SO))
_f32p = np.ctypeslib.ndpointer(np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(np.int32, flags="C_CONTIGUOUS")
_u32p = np.ctypeslib.ndpointer(np.uint32, flags="C_CONTIGUOUS")
_u16p = np.ctypeslib.ndpointer(np.uint16, flags="C_CONTIGUOUS")
_f64p = np.ctypeslib.ndpointer(np.float64, flags="C_CONTIGUOUS")
_lib.oracle_vecadd.argtypes = [_f32p, _f32p, _f32p, C.c_uint64]
_lib.oracle_triad.argtypes = [_f32p, _f32p, _f32p, C.c_float, C.c_uint64]
_lib.oracle_checksum_u32.argtypes = [_u32p, C.c_uint64]
_lib.oracle_checksum_u32.restype = C.c_uint64
_lib.oracle_radix_sort_i32.argtypes = [_i32p, _i32p, C.c_uint64]
_lib.oracle_qsort_i32.argtypes = [_i32p, C.c_uint64]
_lib.oracle_digit_hist.argtypes = [_i32p, C.c_uint64, C.c_int, _u32p]
_lib.oracle_f32_to_bf16.argtypes = [C.c_float]
_lib.oracle_f32_to_bf16.restype = C.c_uint16
_lib.oracle_gemm_bf16_rows.argtypes = [_f64p, _u16p, _u16p, C.c_uint32, C.c_uint32, _u32p, C.c_uint32]


def vecadd(a: np.ndarray, b: np.ndarray) -> np.ndarray:
    c = np.empty_like(a)
    _lib.oracle_vecadd(c, a, b, a.size)
    return c


def triad(b: np.ndarray, c: np.ndarray, s: float) -> np.ndarray:
    a = np.empty_like(b)
    _lib.oracle_triad(a, b, c, s, b.size)
    return a


def checksum_u32(x: np.ndarray) -> int:
    x = np.ascontiguousarray(x).view(np.uint32)
    return int(_lib.oracle_checksum_u32(x, x.size))


def radix_sort_i32(keys: np.ndarray) -> np.ndarray:
    k = np.array(keys, dtype=np.int32, copy=True)
    tmp = np.empty_like(k)
    _lib.oracle_radix_sort_i32(k, tmp, k.size)
    return k


def qsort_i32(keys: np.ndarray) -> np.ndarray:
    k = np.array(keys, dtype=np.int32, copy=True)
    _lib.oracle_qsort_i32(k, k.size)
    return k


def digit_hist(keys: np.ndarray, digit: int) -> np.ndarray:
    h = np.zeros(256, dtype=np.uint32)
    _lib.oracle_digit_hist(np.ascontiguousarray(keys, dtype=np.int32), keys.size, digit, h)
    return h


def f32_to_bf16(x: float) -> int:
    return int(_lib.oracle_f32_to_bf16(x))


def gemm_bf16_rows(a_bits: np.ndarray, b_bits: np.ndarray, rows: np.ndarray) -> np.ndarray:
    """fp64 product rows of A[M,K] * B[N,K]^T from bf16 bit patterns (uint16 arrays)."""
    M, K = a_bits.shape
    N, K2 = b_bits.shape
    assert K == K2
    rows = np.ascontiguousarray(rows, dtype=np.uint32)
    out = np.empty((rows.size, N), dtype=np.float64)
    _lib.oracle_gemm_bf16_rows(out, np.ascontiguousarray(a_bits), np.ascontiguousarray(b_bits), N, K, rows, rows.size)
    return out
