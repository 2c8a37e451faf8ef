"""Every symbol the public headers declare is exported by the library that is said to provide it (load only;
no compute calls, no GPU needed), and the record layouts in wire.h have the sizes the reference's structs have."""
import ctypes
import re
import struct
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
INC = ROOT / "include"


def declared(header: Path, pattern: str) -> set[str]:
    return set(re.findall(pattern, header.read_text()))


@pytest.fixture(scope="module", autouse=True)
def built():
    if not (LIB / "libpreempt.so").exists():
        from xsched_b200 import build
        build.build_all()


def test_libpreempt_exports_the_24_reference_symbols():
    names = declared(INC / "xsched" / "xsched.h", r"^XResult\s+((?:XQueue|HwQueue|HwCommand|XHint)\w+)\s*\(")
    names |= set(re.findall(r"XResult\s+((?:XQueue|HwQueue|HwCommand|XHint)\w+)\s*\(", (INC / "xsched" / "xsched.h").read_text()))
    assert len(names) == 24, sorted(names)
    lib = ctypes.CDLL(str(LIB / "libpreempt.so"))
    missing = [n for n in sorted(names) if not hasattr(lib, n)]
    assert not missing, missing


def test_libhalhost_and_libhalcuda_exports():
    host = set(re.findall(r"XResult\s+(HostLane\w+)\s*\(", (INC / "xsched" / "host" / "hal.h").read_text()))
    lib = ctypes.CDLL(str(LIB / "libhalhost.so"))
    assert host and not [n for n in host if not hasattr(lib, n)]
    # libhalcuda.so needs the CUDA runtime's driver only when a queue is created: loading it must work without a GPU
    cuda = set(re.findall(r"XResult\s+(Cuda\w+)\s*\(", (INC / "xsched" / "cuda" / "hal.h").read_text()))
    lib = ctypes.CDLL(str(LIB / "libhalcuda.so"))
    assert {"CudaQueueCreate", "CudaQueueGet"} <= cuda
    assert not [n for n in cuda if not hasattr(lib, n)]
    # error behaviour that needs no device: null out-pointer and the NULL stream (reference: level1/cuda_queue.cpp:66-98)
    h = ctypes.c_uint64(0)
    assert lib.CudaQueueCreate(None, ctypes.c_void_p(1)) == 2          # kXSchedErrorInvalidValue
    assert lib.CudaQueueCreate(ctypes.byref(h), None) == 5             # kXSchedErrorNotSupported
    assert lib.CudaQueueGet(ctypes.byref(h), None) == 5
    assert lib.CudaQueueGet(ctypes.byref(h), ctypes.c_void_p(0x1234)) == 3   # kXSchedErrorNotFound


def test_shim_exports_the_driver_surface():
    shim = LIB / "libshimcuda.so"
    assert shim.exists()
    import subprocess
    out = subprocess.run(["nm", "-D", "--defined-only", str(shim)], capture_output=True, text=True, check=True).stdout
    syms = {l.split()[-1] for l in out.splitlines() if " T " in l}
    for must in ("cuInit", "cuLaunchKernel", "cuLaunchKernelEx", "cuMemcpyAsync", "cuMemcpyHtoDAsync_v2", "cuEventRecord", "cuStreamSynchronize",
                 "cuGetProcAddress", "cuGetProcAddress_v2", "cuMemAlloc_v2", "cuCtxGetCurrent", "cuStreamCreateWithPriority", "XSchedShimMarker" if False else "cuMemFree_v2"):
        assert must in syms, must
    assert len([s for s in syms if s.startswith("cu")]) > 550
    assert "XSchedShimMarker" in out


def test_wire_record_sizes_match_the_reference_structs():
    from oracle import sched_oracle as so
    assert len(so.ev_proc_create(1)) == 264 and len(so.ev_proc_destroy(1)) == 8
    assert len(so.ev_xq_create(1, 2, 3)) == 48 and len(so.ev_xq_ready(1, 2, 3)) == 24 and len(so.ev_xq_idle(1, 2)) == 16
    assert len(so.ev_hint_priority(1, 2, 3)) == 16 + 24 and len(so.ev_hint_laxity(1, 2, 3, 4, 5)) == 16 + 32
    # operation header: {u64 id, i32 type, i32 pid, u64 size, u64 running, u64 suspended} then handles
    assert struct.calcsize("<Qii QQQ") == 40


def test_pk_header_and_python_face_agree():
    """Every symbol and every enumerator of include/xsched_b200/pk.h that the ctypes face names has the header's value:
    the flags (including the two that choose the GEMM's form), the status and result codes, the exported functions."""
    import re
    from xsched_b200 import pk
    text = (ROOT / "include" / "xsched_b200" / "pk.h").read_text()
    enums = {m.group(1): int(m.group(2), 0) for m in re.finditer(r"\b(XPK_[A-Z0-9_]+)\s*=\s*(0x[0-9a-fA-F]+|\d+)", text)}
    want = {"XPK_FLAG_NONE": pk.FLAG_NONE, "XPK_FLAG_NON_PREEMPTIBLE": pk.FLAG_NON_PREEMPTIBLE, "XPK_FLAG_ABORT_INFLIGHT": pk.FLAG_ABORT_INFLIGHT,
            "XPK_FLAG_GEMM_ONE_CTA": pk.FLAG_GEMM_ONE_CTA, "XPK_FLAG_GEMM_CTA_PAIR": pk.FLAG_GEMM_CTA_PAIR,
            "XPK_KIND_TRIAD": pk.KIND_TRIAD, "XPK_KIND_VECADD": pk.KIND_VECADD, "XPK_KIND_SORT": pk.KIND_SORT, "XPK_KIND_GEMM": pk.KIND_GEMM}
    for name, value in want.items():
        assert enums.get(name) == value, (name, enums.get(name), value)
    assert pk.FLAG_GEMM_ONE_CTA & pk.FLAG_GEMM_CTA_PAIR == 0
    declared = set(re.findall(r"\b(xpk[A-Z][A-Za-z0-9]+)\s*\(", text))
    assert declared == set(pk.EXPORTS), declared ^ set(pk.EXPORTS)
    for sym in pk.EXPORTS:
        assert hasattr(pk.lib, sym), sym
