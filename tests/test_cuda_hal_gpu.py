"""CUDA HAL end to end on a GPU: XQueue C API -> CudaQueue (level 1 window / level 2 flag) -> xpk kernels,
driven through the native worker.  The worker spoils every output buffer before each iteration and compares
it with an unpreempted run's after it (order-sensitive hashes), so a tile that a flushed-and-replayed
command never wrote fails the run; one test spoils a sample on purpose to show that the check can fail."""
import json
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
WORKER = ROOT / "xsched_b200" / "lib" / "xbench_worker"


def run(*args, env_extra=None, timeout=300, expect_rc=0):
    env = dict(os.environ, XLOG_LEVEL="WARN")
    env.pop("XSCHED_SCHEDULER", None)
    env.pop("XSCHED_POLICY", None)
    env.update(env_extra or {})
    r = subprocess.run([str(WORKER), *map(str, args)], capture_output=True, text=True, env=env, timeout=timeout)
    assert r.returncode == expect_rc, f"rc={r.returncode}\n{r.stdout[-1500:]}\n{r.stderr[-1500:]}"
    return [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]


@pytest.mark.parametrize("kernel,extra", [("gemm", ["--M", 4096, "--N", 4096, "--K", 4096]), ("triad", ["--n", 1 << 27]),
                                          ("sort", ["--n", 1 << 24])])
@pytest.mark.parametrize("level", [1, 2])
def test_suspend_resume_keeps_output_bit_exact(kernel, extra, level):
    out = run("--role", "preempt-latency", "--kernel", kernel, "--level", level, "--count", 60, *extra)[-1]
    assert out["bit_exact"] is True and out["mismatched_outputs"] == 0
    assert out["n"] == 60 and out["rounds_checked"] > 5
    if level == 2:
        assert out["deactivations"] == 60
        assert out["relaunches"] > 0          # at least one kernel was cut and resumed from its cursor
        assert out["preempted_outputs_checked"] > 0      # and the output of such a run was looked at


@pytest.mark.parametrize("kernel,extra", [("gemm", ["--M", 2048, "--N", 2048, "--K", 2048]), ("triad", ["--n", 1 << 26])])
def test_output_check_sees_a_spoiled_sample(kernel, extra):
    """One 32-byte sample of one output is overwritten before it is verified — what a tile that was never
    written leaves behind: the worker must report a mismatch and exit non-zero."""
    out = run("--role", "preempt-latency", "--kernel", kernel, "--level", 2, "--count", 20, "--tamper-at", 2, *extra, expect_rc=6)[-1]
    assert out["bit_exact"] is False and out["mismatched_outputs"] == 1
    hp_lp = run("--role", "lp", "--kernel", kernel, "--level", 2, "--duration-s", 1, "--warmup-s", 0.2, "--tamper-at", 3, *extra, expect_rc=6)[-1]
    assert hp_lp["bit_exact"] is False and hp_lp["mismatched_iters"] == 1


def test_two_queues_in_process_hpf_level2():
    hp, lp = run("--role", "both", "--kernel", "gemm", "--level", 2, "--count", 100, "--period-us", 5000, "--duration-s", 2,
                 "--hp-n", 1 << 24)
    assert hp["verified"] is True and hp["n"] >= 50
    assert lp["bit_exact"] is True and lp["iters"] > 10
    assert lp["deactivations"] > 10 and lp["relaunches"] > 0
    assert lp["verified_iters"] >= lp["iters"] and lp["verified_preempted_iters"] > 0 and lp["mismatched_iters"] == 0


def test_level1_window_only():
    hp, lp = run("--role", "both", "--kernel", "gemm", "--level", 1, "--count", 40, "--period-us", 10000, "--duration-s", 1,
                 "--hp-n", 1 << 24, "--M", 2048, "--N", 2048, "--K", 2048)
    assert hp["verified"] is True
    assert lp["bit_exact"] is True and lp["deactivations"] == 0
