"""`from xsched.cuda import XSchedCuda` — Python face of libhalcuda.so.

CudaQueueCreate / CudaQueueGet as in the reference's package (platforms/cuda/python/xsched/cuda/__init__.py);
CudaQueueGetPreemptFlag, CudaXpkCommandCreate and CudaQueueGetStats are this implementation's additions for
level-2 preemption with the preemptible kernel library (include/xsched/cuda/hal.h).
"""
import ctypes as _C

from xsched import HwCommandHandle, HwQueueHandle, XResult, _bind, _u64, load_library  # noqa: F401

CUstream = int


class CudaQueueStats(_C.Structure):
    _fields_ = [(n, _C.c_uint64) for n in ("launched", "completed", "window_stalls", "deactivations", "relaunches", "last_preempt_ns")]


_dll = load_library("libhalcuda.so")
_dll.CudaQueueGetStats.restype = _C.c_int32
_dll.CudaQueueGetStats.argtypes = [_u64, _C.POINTER(CudaQueueStats)]


def _stats(hwq: HwQueueHandle):
    st = CudaQueueStats()
    res = _dll.CudaQueueGetStats(hwq, _C.byref(st))
    return XResult(res), {n: int(getattr(st, n)) for n, _ in CudaQueueStats._fields_}


XSchedCuda = type("XSchedCuda", (), {
    "dll": _dll,
    "CudaQueueCreate": _bind(_dll, "CudaQueueCreate", (_C.c_int64,), _u64, int, False),
    "CudaQueueGet": _bind(_dll, "CudaQueueGet", (_C.c_int64,), _u64, int, False),
    "CudaQueueGetPreemptFlag": _bind(_dll, "CudaQueueGetPreemptFlag", (_u64,), _C.c_void_p, lambda v: int(v or 0), True),
    "CudaXpkCommandCreate": _bind(_dll, "CudaXpkCommandCreate", (_C.c_void_p, _C.c_int32), _u64, int, False),
    "CudaQueueGetStats": staticmethod(_stats),
})
