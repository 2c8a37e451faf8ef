"""CPU checks of the kernel-arithmetic oracle against independent implementations, plus the
exported-symbol contract of libxpk.so (no GPU needed, no compute calls)."""
import ctypes
import re
from pathlib import Path

import numpy as np
import pytest

from oracle import kernels as ok

ROOT = Path(__file__).resolve().parent.parent


def test_vecadd_is_plain_fp32_add():
    rng = np.random.default_rng(0)
    a = rng.uniform(-1, 1, 10001).astype(np.float32)
    b = rng.uniform(-1, 1, 10001).astype(np.float32)
    assert np.array_equal(ok.vecadd(a, b), a + b)


def test_triad_is_single_rounding_fma():
    rng = np.random.default_rng(1)
    b = rng.uniform(-1, 1, 200003).astype(np.float32)
    c = rng.uniform(-1, 1, 200003).astype(np.float32)
    s = np.float32(1.7)
    got = ok.triad(b, c, float(s))
    # s*c is exact in fp64; adding b rounds once to 53 bits, then once more to fp32.  The second
    # rounding can differ from a true fma only on exact ties of the first, which is very rare.
    approx = (np.float64(s) * c.astype(np.float64) + b.astype(np.float64)).astype(np.float32)
    diff = got != approx
    assert diff.mean() < 1e-5
    if diff.any():
        ulp = np.abs(got[diff].view(np.int32) - approx[diff].view(np.int32))
        assert ulp.max() <= 1
    # and it is NOT the two-rounding expression in general
    two = b + s * c
    assert (got != two).any()
    # exact known answers
    one = np.array([1.0], np.float32)
    assert ok.triad(one, np.array([2.0 ** -24], np.float32), 1.0)[0] == np.float32(1.0)
    assert ok.triad(np.array([-1.0], np.float32), np.array([1.0 + 2.0 ** -23], np.float32), 1.0 + 2.0 ** -23)[0] \
        == np.float32(2.0 ** -22 + 2.0 ** -46)


@pytest.mark.parametrize("n", [0, 1, 2, 255, 256, 8193, 100003])
def test_radix_sort_matches_qsort_and_numpy(n):
    rng = np.random.default_rng(n)
    k = rng.integers(-2**31, 2**31, size=n, dtype=np.int64).astype(np.int32)
    r = ok.radix_sort_i32(k)
    assert np.array_equal(r, ok.qsort_i32(k))
    assert np.array_equal(r, np.sort(k, kind="stable"))


def test_radix_sort_edge_values():
    k = np.array([0, -1, 2**31 - 1, -2**31, 1, -2**31, 2**31 - 1, 0], dtype=np.int32)
    assert np.array_equal(ok.radix_sort_i32(k), np.sort(k))
    h = ok.digit_hist(k, 3)
    assert h.sum() == k.size and h[0] == 2 and h[255] == 2     # sign-flipped top byte


def test_bf16_rounding_and_gemm_rows():
    import struct
    for f in (1.0, -2.5, 3.14159, 1e-3, 65504.0, 1.00390625, 1.01171875):
        bits = struct.unpack("<I", struct.pack("<f", f))[0]
        want = (bits + 0x7FFF + ((bits >> 16) & 1)) >> 16
        assert ok.f32_to_bf16(f) == want
    rng = np.random.default_rng(2)
    M, N, K = 16, 24, 96
    a = (rng.standard_normal((M, K)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    b = (rng.standard_normal((N, K)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16)
    af = (a.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    bf = (b.astype(np.uint32) << 16).view(np.float32).astype(np.float64)
    rows = np.array([0, 5, 15], dtype=np.uint32)
    got = ok.gemm_bf16_rows(a, b, rows)
    assert np.allclose(got, (af @ bf.T)[rows], rtol=1e-12, atol=1e-12)


def test_libxpk_exports_every_declared_symbol():
    header = (ROOT / "include" / "xsched_b200" / "pk.h").read_text()
    declared = set(re.findall(r"\b(xpk[A-Z]\w+)\s*\(", header))
    so = ROOT / "xsched_b200" / "lib" / "libxpk.so"
    assert so.exists(), "libxpk.so not built (python -m xsched_b200.build)"
    lib = ctypes.CDLL(str(so))
    missing = [s for s in sorted(declared) if not hasattr(lib, s)]
    assert not missing, missing
    assert len(declared) >= 18
