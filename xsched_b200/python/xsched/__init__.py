"""`import xsched` — Python face of libpreempt.so (the XQueue / HwQueue / XHint C entry points).

Same names, argument order and return conventions as the reference's package (python/xsched/__init__.py):
every call is a static method of `XSched`; calls that fill an out-parameter return `(XResult, value)`.
The methods are generated from one signature table.  Put this directory on PYTHONPATH and the directory
holding libpreempt.so on LD_LIBRARY_PATH (or set XSCHED_LIB_DIR); the library is also looked for next to
this package (../../lib).
"""
from __future__ import annotations

import ctypes as _C
import os as _os
from enum import IntEnum
from pathlib import Path as _Path

XDevice = XDeviceId = XQueueHandle = HwQueueHandle = HwCommandHandle = int
Priority = Utilization = Timeslice = Laxity = Deadline = int


XResult = IntEnum("XResult", dict(kXSchedSuccess=0, kXSchedErrorHardware=1, kXSchedErrorInvalidValue=2, kXSchedErrorNotFound=3,
                                  kXSchedErrorNotAllowed=4, kXSchedErrorNotSupported=5, kXSchedErrorBadResponse=6, kXSchedErrorUnknown=999))
XPlatform = IntEnum("XPlatform", dict(kPlatformUnknown=0, kPlatformVPI=1, kPlatformCUDA=2, kPlatformCUDLA=3, kPlatformHIP=4,
                                      kPlatformAscend=5, kPlatformOpenCL=6, kPlatformLevelZero=7))
XDeviceType = IntEnum("XDeviceType", dict(kDeviceTypeUnknown=0, kDeviceTypeCPU=1, kDeviceTypeGPU=2, kDeviceTypeNPU=3, kDeviceTypeFPGA=4,
                                          kDeviceTypeASIC=5, kDeviceTypeMCA=6))
XPreemptLevel = IntEnum("XPreemptLevel", dict(kPreemptLevelUnknown=0, kPreemptLevelBlock=1, kPreemptLevelDeactivate=2,
                                              kPreemptLevelInterrupt=3, kPreemptLevelMax=4))
XQueueState = IntEnum("XQueueState", dict(kQueueStateUnknown=0, kQueueStateIdle=1, kQueueStateReady=2))
XQueueFeature = IntEnum("XQueueFeature", dict(kQueueFeatureNone=0, kQueueFeatureAsyncSubmit=1, kQueueFeatureDynamicLevel=2,
                                              kQueueFeatureDynamicThreshold=4, kQueueFeatureDynamicBatchSize=8, kQueueFeatureSyncSuspend=16,
                                              kQueueFeatureResumeDropCommands=32, kQueueFeatureMaskAll=-1))
XQueueCreateFlag = IntEnum("XQueueCreateFlag", dict(kQueueCreateFlagNone=0, kQueueCreateFlagBlockingSubmit=1, kQueueCreateFlagMaskAll=-1))
XQueueSuspendFlag = IntEnum("XQueueSuspendFlag", dict(kQueueSuspendFlagNone=0, kQueueSuspendFlagSyncHwQueue=1, kQueueSuspendFlagWaitAll=2,
                                                      kQueueSuspendFlagWaitIdle=4, kQueueSuspendFlagMaskAll=-1))
XQueueResumeFlag = IntEnum("XQueueResumeFlag", dict(kQueueResumeFlagNone=0, kQueueResumeFlagDropCommands=1, kQueueResumeFlagMaskAll=-1))
XSchedulerType = IntEnum("XSchedulerType", dict(kSchedulerUnknown=0, kSchedulerAppManaged=1, kSchedulerLocal=2, kSchedulerGlobal=3, kSchedulerMax=4))
XPolicyType = IntEnum("XPolicyType", dict(
    kPolicyUnknown=0, kPolicyHighestPriorityFirst=1, kPolicyHeterogeneousHighestPriorityFirst=2, kPolicyCPUHighestPriorityFirst=3,
    kPolicyUtilizationPartition=4, kPolicyProcessUtilizationPartition=5, kPolicyStrictProcessUtilizationPartition=6,
    kPolicyKEarliestDeadlineFirst=7, kPolicyLaxity=8, kPolicyActiveWindowFirst=9, kPolicyCompletelyFairScheduler=10,
    kPolicyMultiLevelFeedbackQueue=11, kPolicyMax=12))

PRIORITY_NO_EXECUTE, PRIORITY_MIN, PRIORITY_DEFAULT, PRIORITY_MAX = -256, -255, 0, 255
UTILIZATION_MIN, UTILIZATION_DEFAULT, UTILIZATION_MAX = 0, 100, 100
TIMESLICE_MIN, TIMESLICE_DEFAULT, TIMESLICE_MAX, TIMESLICE_UNLIMITED = 100, 5000, 10_000_000, 0xFFFFFFFFFFFFFFFF
NO_LAXITY = NO_DEADLINE = -1


def load_library(name: str) -> _C.CDLL:
    """dlopen by name (loader path, as the reference does), else from $XSCHED_LIB_DIR, else from ../../lib."""
    tried = []
    for cand in (name, _os.path.join(_os.environ.get("XSCHED_LIB_DIR", ""), name), str(_Path(__file__).resolve().parents[2] / "lib" / name)):
        try:
            return _C.cdll.LoadLibrary(cand)
        except OSError as e:
            tried.append(f"{cand}: {e}")
    raise RuntimeError(f"failed to load {name} bindings: " + "; ".join(tried))


_u64, _i64, _i32 = _C.c_uint64, _C.c_int64, _C.c_int32
# name -> (ctypes of the inputs, ctype of the out-parameter (first C argument) or None, converter of the out value)
_SIGNATURES = {
    "XQueueCreate": ((_u64, _i64, _i64), _u64, int),
    "XQueueDestroy": ((_u64,), None, None),
    "XQueueGet": ((_u64,), _u64, int),
    "XQueueSetPreemptLevel": ((_u64, _i32), None, None),
    "XQueueSetLaunchConfig": ((_u64, _i64, _i64), None, None),
    "XQueueSubmit": ((_u64, _u64), None, None),
    "XQueueWait": ((_u64, _u64), None, None),
    "XQueueWaitAll": ((_u64,), None, None),
    "XQueueSuspend": ((_u64, _i64), None, None),
    "XQueueResume": ((_u64, _i64), None, None),
    "HwQueueDestroy": ((_u64,), None, None),
    "HwQueueLaunch": ((_u64, _u64), None, None),
    "HwQueueSynchronize": ((_u64,), None, None),
    "HwCommandDestroy": ((_u64,), None, None),
    "XHintSetScheduler": ((_i32, _i32), None, None),
    "XHintPriority": ((_u64, _i32), None, None),
    "XHintUtilization": ((_u64, _i32), None, None),
    "XHintTimeslice": ((_i64,), None, None),
    "XHintLaxity": ((_u64, _i64, _i32, _i32), None, None),
    "XHintDeadline": ((_u64, _i64), None, None),
    "XHintKDeadline": ((_C.c_size_t,), None, None),
}
# out-parameter LAST in the C signature
_TRAILING_OUT = {
    "XQueueQuery": ((_u64,), _i32, XQueueState),
    "XQueueProfileHwCommandCount": ((_u64,), _i64, int),
}


def _bind(dll, name, ins, out, conv, trailing):
    fn = getattr(dll, name)
    fn.restype = _i32
    if out is None:
        fn.argtypes = list(ins)
        return staticmethod(lambda *a: XResult(fn(*a)))
    fn.argtypes = (list(ins) + [_C.POINTER(out)]) if trailing else ([_C.POINTER(out)] + list(ins))

    def call(*a):
        box = out()
        res = fn(*a, _C.byref(box)) if trailing else fn(_C.byref(box), *a)
        return XResult(res), conv(box.value)
    return staticmethod(call)


def _make(cls_name: str, dll, leading: dict, trailing: dict) -> type:
    members = {n: _bind(dll, n, *sig, False) for n, sig in leading.items()}
    members.update({n: _bind(dll, n, *sig, True) for n, sig in trailing.items()})
    members["dll"] = dll
    return type(cls_name, (), members)


XSched = _make("XSched", load_library("libpreempt.so"), _SIGNATURES, _TRAILING_OUT)
