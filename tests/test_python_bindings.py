"""The `xsched` Python package (xsched_b200/python): same calls and return conventions as the reference's ctypes
package, exercised on the host-only lane; and the reference's OWN package, unmodified, run against this
repository's libpreempt.so (it loads the library by name) must give the same answers."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
REF_PY = Path(os.environ.get("XSCHED_REFERENCE_DIR", "/root/reference")) / "python"

SCRIPT = r"""
import ctypes, json, sys
from xsched import XSched, XResult, XPreemptLevel, XQueueState, XSchedulerType, XPolicyType, XQueueSuspendFlag, XQueueResumeFlag, XQueueCreateFlag
lane = ctypes.CDLL("libhalhost.so")
hwq = ctypes.c_uint64()
assert lane.HostLaneQueueCreate(ctypes.byref(hwq), 0) == 0
out = {}
out["set_sched"] = int(XSched.XHintSetScheduler(XSchedulerType.kSchedulerLocal, XPolicyType.kPolicyHighestPriorityFirst))
res, xq = XSched.XQueueCreate(hwq.value, XPreemptLevel.kPreemptLevelDeactivate, XQueueCreateFlag.kQueueCreateFlagNone)
out["create"] = int(res); assert xq != 0
out["create_again"] = int(XSched.XQueueCreate(hwq.value, XPreemptLevel.kPreemptLevelBlock, 0)[0])
res, xq2 = XSched.XQueueGet(hwq.value)
out["get"] = [int(res), xq2 == xq]
out["get_unknown"] = int(XSched.XQueueGet(0x1234)[0])
out["config"] = int(XSched.XQueueSetLaunchConfig(xq, 4, 2))
out["prio"] = int(XSched.XHintPriority(xq, 3))
out["lax"] = int(XSched.XHintLaxity(xq, 1000, 0, 1))
out["util"] = int(XSched.XHintUtilization(xq, 50))
out["ts"] = int(XSched.XHintTimeslice(5000))
out["ddl"] = int(XSched.XHintDeadline(xq, 10000))
out["kddl"] = int(XSched.XHintKDeadline(2))
cmds = []
for i in range(6):
    c = ctypes.c_uint64()
    assert lane.HostLaneCommandCreate(ctypes.byref(c), ctypes.c_int64(500)) == 0
    cmds.append(c.value)
    out.setdefault("submit", []).append(int(XSched.XQueueSubmit(xq, c.value)))
out["wait_one"] = int(XSched.XQueueWait(xq, cmds[2]))
out["suspend"] = int(XSched.XQueueSuspend(xq, XQueueSuspendFlag.kQueueSuspendFlagSyncHwQueue))
out["resume"] = int(XSched.XQueueResume(xq, XQueueResumeFlag.kQueueResumeFlagNone))
out["wait_all"] = int(XSched.XQueueWaitAll(xq))
res, st = XSched.XQueueQuery(xq)
out["query"] = [int(res), int(st), isinstance(st, XQueueState)]
out["count"] = [int(v) for v in XSched.XQueueProfileHwCommandCount(xq)]
out["level"] = int(XSched.XQueueSetPreemptLevel(xq, XPreemptLevel.kPreemptLevelBlock))
out["sync_hwq"] = int(XSched.HwQueueSynchronize(hwq.value))
out["destroy"] = int(XSched.XQueueDestroy(xq))
out["destroy_again"] = int(XSched.XQueueDestroy(xq))
out["hwq_destroy"] = int(XSched.HwQueueDestroy(hwq.value))
out["types"] = isinstance(res, XResult)
print(json.dumps(out))
"""


def run(pythonpath: Path) -> dict:
    env = dict(os.environ, XLOG_LEVEL="ERRO", PYTHONPATH=str(pythonpath), LD_LIBRARY_PATH=f"{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""))
    env.pop("XSCHED_SCHEDULER", None)
    r = subprocess.run([sys.executable, "-c", SCRIPT], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout.strip().splitlines()[-1])


def test_package_calls_and_result_codes():
    got = run(ROOT / "xsched_b200" / "python")
    assert got["create"] == 0 and got["get"] == [0, True] and got["get_unknown"] == 3
    assert got["config"] == 0
    assert got["submit"] == [0] * 6 and got["wait_all"] == 0
    assert got["wait_one"] == 3                          # a submitted command's handle is gone (ownership passed to the queue)
    assert got["suspend"] == 0 and got["resume"] == 0
    assert got["query"] == [0, 1, True]                  # idle after WaitAll, returned as the enum
    assert got["count"] == [0, 6]
    assert got["destroy"] == 0 and got["destroy_again"] == 3 and got["types"] is True


@pytest.mark.skipif(not REF_PY.exists(), reason="reference tree not present")
def test_reference_package_runs_unmodified_on_this_library():
    assert run(REF_PY) == run(ROOT / "xsched_b200" / "python")


def test_cuda_package_exposes_the_hal_entry_points():
    env = dict(os.environ, PYTHONPATH=str(ROOT / "xsched_b200" / "python"), LD_LIBRARY_PATH=f"{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""))
    code = ("from xsched.cuda import XSchedCuda\n"
            "print(all(hasattr(XSchedCuda, n) for n in ('CudaQueueCreate','CudaQueueGet','CudaQueueGetPreemptFlag','CudaXpkCommandCreate','CudaQueueGetStats')))\n"
            "r, h = XSchedCuda.CudaQueueGet(0)\nprint(int(r), h)\n")
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = r.stdout.split()
    assert lines[0] == "True" and int(lines[1]) == 5          # the default stream is not supported (no GPU needed to ask)
