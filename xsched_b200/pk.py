"""ctypes face of libxpk.so (include/xsched_b200/pk.h): preemptible persistent kernels.

torch is used by callers for device memory and streams only; every kernel that runs is one of
the hand-written sm_100a kernels in xsched_b200/csrc/kernels.  If the shared library is missing
the import fails — there is no fallback path.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass

from . import LIB_DIR

_LIB_PATH = LIB_DIR / "libxpk.so"
if not _LIB_PATH.exists():
    raise ImportError(f"{_LIB_PATH} not built; run `python -m xsched_b200.build` (needs nvcc)")
lib = C.CDLL(str(_LIB_PATH))

SUCCESS = 0
STATUS_IDLE, STATUS_RUNNING, STATUS_COMPLETED, STATUS_PREEMPTED, STATUS_ERROR = range(5)
KIND_TRIAD, KIND_VECADD, KIND_SORT, KIND_GEMM = 1, 2, 3, 4
FLAG_NONE, FLAG_NON_PREEMPTIBLE, FLAG_ABORT_INFLIGHT, FLAG_GEMM_ONE_CTA, FLAG_GEMM_CTA_PAIR = 0, 1, 2, 4, 8

#: every symbol include/xsched_b200/pk.h declares
EXPORTS = [
    "xpkDeviceSmCount", "xpkResultString", "xpkFlagCreate", "xpkFlagDestroy", "xpkFlagSet",
    "xpkTaskCreateTriad", "xpkTaskCreateVecAdd", "xpkSortScratchBytes", "xpkTaskCreateSort",
    "xpkTaskCreateGemm", "xpkTaskLaunch", "xpkTaskQuery", "xpkTaskWait", "xpkTaskReset",
    "xpkTaskFlag", "xpkTaskKind", "xpkTaskDestroy", "xpkLaunchCount", "xpkSortNoAlloc", "xpkTaskTimes",
    "xpkFlagAttachRelay", "xpkFlagDetachRelay",
]


class TaskInfo(C.Structure):
    _fields_ = [("status", C.c_uint32), ("error", C.c_uint32), ("tiles_done", C.c_uint64),
                ("tiles_total", C.c_uint64), ("launches", C.c_uint64), ("preemptions", C.c_uint64)]


_vp, _u32, _u64 = C.c_void_p, C.c_uint32, C.c_uint64
lib.xpkResultString.restype = C.c_char_p
lib.xpkResultString.argtypes = [C.c_int]
lib.xpkDeviceSmCount.argtypes = [C.POINTER(C.c_int)]
lib.xpkFlagCreate.argtypes = [C.POINTER(_vp)]
lib.xpkFlagDestroy.argtypes = [_vp]
lib.xpkFlagSet.argtypes = [_vp, _u32, _vp]
lib.xpkFlagAttachRelay.argtypes = [_vp, C.POINTER(_vp)]
lib.xpkFlagDetachRelay.argtypes = [_vp, _vp]
lib.xpkTaskCreateTriad.argtypes = [C.POINTER(_vp), _vp, _vp, _vp, C.c_float, _u64, _u32, _u32, _vp]
lib.xpkTaskCreateVecAdd.argtypes = [C.POINTER(_vp), _vp, _vp, _vp, _u64, _u32, _u32, _vp]
lib.xpkSortScratchBytes.restype = C.c_size_t
lib.xpkSortScratchBytes.argtypes = [_u64]
lib.xpkTaskCreateSort.argtypes = [C.POINTER(_vp), _vp, _vp, _vp, _u64, _u32, _vp]
lib.xpkTaskCreateGemm.argtypes = [C.POINTER(_vp), _vp, _vp, _vp, _u32, _u32, _u32, _u32, _vp]
lib.xpkTaskLaunch.argtypes = [_vp, _vp, C.c_int]
lib.xpkTaskQuery.argtypes = [_vp, C.POINTER(TaskInfo)]
lib.xpkTaskWait.argtypes = [_vp, _u64, C.POINTER(TaskInfo)]
lib.xpkTaskReset.argtypes = [_vp, _vp]
lib.xpkTaskTimes.argtypes = [_vp, C.POINTER(_u64), C.POINTER(_u64)]
lib.xpkTaskFlag.argtypes = [_vp, C.POINTER(_vp)]
lib.xpkTaskKind.argtypes = [_vp, C.POINTER(_u32)]
lib.xpkTaskDestroy.argtypes = [_vp]
lib.xpkLaunchCount.restype = _u64
lib.xpkSortNoAlloc.argtypes = [_vp, _vp, _u64, _vp]
SORT_NOALLOC_MAX_KEYS = 4 << 20


class XpkError(RuntimeError):
    def __init__(self, code: int, what: str):
        super().__init__(f"{what}: {lib.xpkResultString(code).decode()} ({code})")
        self.code = code


def _check(code: int, what: str) -> None:
    if code != SUCCESS:
        raise XpkError(code, what)


def sm_count() -> int:
    n = C.c_int(0)
    _check(lib.xpkDeviceSmCount(C.byref(n)), "xpkDeviceSmCount")
    return n.value


def launch_count() -> int:
    return int(lib.xpkLaunchCount())


def sort_scratch_bytes(n: int) -> int:
    return int(lib.xpkSortScratchBytes(n))


def sort_no_alloc(keys, tmp, stream: int) -> None:
    """In-place ascending sort of the int32 tensor `keys` through xpkSortNoAlloc (no allocation at all;
    at most SORT_NOALLOC_MAX_KEYS keys; calls on one device must not overlap on the GPU)."""
    _check(lib.xpkSortNoAlloc(keys.data_ptr(), tmp.data_ptr(), keys.numel(), stream), "xpkSortNoAlloc")


class Flag:
    """One 32-bit preempt flag in device memory, shareable between tasks."""

    def __init__(self):
        p = _vp()
        _check(lib.xpkFlagCreate(C.byref(p)), "xpkFlagCreate")
        self.ptr = p.value

    def set(self, value: int, ctrl_stream: int = 0) -> None:
        _check(lib.xpkFlagSet(self.ptr, value, ctrl_stream), "xpkFlagSet")

    def attach_relay(self):
        """Give the flag an early-warning word in mapped host memory; returns it as a ctypes c_uint32 the caller
        stores to (non-zero just before raising the flag, zero before lowering it)."""
        p = _vp()
        _check(lib.xpkFlagAttachRelay(self.ptr, C.byref(p)), "xpkFlagAttachRelay")
        self.relay = p.value
        return C.c_uint32.from_address(p.value)

    def destroy(self) -> None:
        if self.ptr:
            if getattr(self, "relay", None):
                lib.xpkFlagDetachRelay(self.ptr, self.relay)
                self.relay = None
            lib.xpkFlagDestroy(self.ptr)
            self.ptr = None


@dataclass
class Info:
    status: int
    error: int
    tiles_done: int
    tiles_total: int
    launches: int
    preemptions: int


class Task:
    """Handle of one preemptible task.  Keep the tensors whose pointers were passed alive."""

    def __init__(self, handle: int, keepalive=()):
        self.handle = handle
        self._keep = keepalive

    # -- constructors -------------------------------------------------------------------
    @staticmethod
    def triad(a, b, c, s: float, tile_elems: int = 0, flags: int = 0, flag: Flag | None = None) -> "Task":
        h = _vp()
        _check(lib.xpkTaskCreateTriad(C.byref(h), a.data_ptr(), b.data_ptr(), c.data_ptr(), s, a.numel(),
                                      tile_elems, flags, flag.ptr if flag else None), "xpkTaskCreateTriad")
        return Task(h.value, (a, b, c, flag))

    @staticmethod
    def vecadd(c, a, b, tile_elems: int = 0, flags: int = 0, flag: Flag | None = None) -> "Task":
        h = _vp()
        _check(lib.xpkTaskCreateVecAdd(C.byref(h), c.data_ptr(), a.data_ptr(), b.data_ptr(), c.numel(),
                                       tile_elems, flags, flag.ptr if flag else None), "xpkTaskCreateVecAdd")
        return Task(h.value, (a, b, c, flag))

    @staticmethod
    def sort(keys, tmp, scratch, flags: int = 0, flag: Flag | None = None) -> "Task":
        h = _vp()
        _check(lib.xpkTaskCreateSort(C.byref(h), keys.data_ptr(), tmp.data_ptr(), scratch.data_ptr(), keys.numel(),
                                     flags, flag.ptr if flag else None), "xpkTaskCreateSort")
        return Task(h.value, (keys, tmp, scratch, flag))

    @staticmethod
    def gemm(c, a, b, flags: int = 0, flag: Flag | None = None) -> "Task":
        """c[M,N] = a[M,K] @ b[N,K].T, all bf16 row-major contiguous."""
        M, K = a.shape
        N, K2 = b.shape
        assert K == K2 and tuple(c.shape) == (M, N)
        h = _vp()
        _check(lib.xpkTaskCreateGemm(C.byref(h), c.data_ptr(), a.data_ptr(), b.data_ptr(), M, N, K, flags,
                                     flag.ptr if flag else None), "xpkTaskCreateGemm")
        return Task(h.value, (a, b, c, flag))

    # -- control ------------------------------------------------------------------------
    def launch(self, stream: int, sm_limit: int = 0) -> None:
        _check(lib.xpkTaskLaunch(self.handle, stream, sm_limit), "xpkTaskLaunch")

    def query(self) -> Info:
        ti = TaskInfo()
        _check(lib.xpkTaskQuery(self.handle, C.byref(ti)), "xpkTaskQuery")
        return Info(ti.status, ti.error, ti.tiles_done, ti.tiles_total, ti.launches, ti.preemptions)

    def wait(self, timeout_us: int = 30_000_000) -> Info:
        ti = TaskInfo()
        _check(lib.xpkTaskWait(self.handle, timeout_us, C.byref(ti)), "xpkTaskWait")
        return Info(ti.status, ti.error, ti.tiles_done, ti.tiles_total, ti.launches, ti.preemptions)

    def reset(self, stream: int) -> None:
        _check(lib.xpkTaskReset(self.handle, stream), "xpkTaskReset")

    def flag_ptr(self) -> int:
        p = _vp()
        _check(lib.xpkTaskFlag(self.handle, C.byref(p)), "xpkTaskFlag")
        return p.value

    def set_flag(self, value: int, ctrl_stream: int = 0) -> None:
        _check(lib.xpkFlagSet(self.flag_ptr(), value, ctrl_stream), "xpkFlagSet")

    def destroy(self) -> None:
        if self.handle:
            lib.xpkTaskDestroy(self.handle)
            self.handle = None
            self._keep = ()
