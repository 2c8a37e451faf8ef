"""CUDA HAL end to end on a GPU: XQueue C API -> CudaQueue (level 1 window / level 2 flag) -> xpk kernels,
driven through the native worker.  Every run re-checks that the low-priority output is bit-identical
to an unpreempted run (order-sensitive checksum of the whole output)."""
import json
import os
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
WORKER = ROOT / "xsched_b200" / "lib" / "xbench_worker"


def run(*args, env_extra=None, timeout=300):
    env = dict(os.environ, XLOG_LEVEL="WARN")
    env.pop("XSCHED_SCHEDULER", None)
    env.pop("XSCHED_POLICY", None)
    env.update(env_extra or {})
    r = subprocess.run([str(WORKER), *map(str, args)], capture_output=True, text=True, env=env, timeout=timeout)
    assert r.returncode == 0, f"rc={r.returncode}\n{r.stdout[-1500:]}\n{r.stderr[-1500:]}"
    return [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]


@pytest.mark.parametrize("kernel,extra", [("gemm", ["--M", 4096, "--N", 4096, "--K", 4096]), ("triad", ["--n", 1 << 27]),
                                          ("sort", ["--n", 1 << 24])])
@pytest.mark.parametrize("level", [1, 2])
def test_suspend_resume_keeps_output_bit_exact(kernel, extra, level):
    out = run("--role", "preempt-latency", "--kernel", kernel, "--level", level, "--count", 60, *extra)[-1]
    assert out["bit_exact"] is True
    assert out["n"] == 60
    if level == 2:
        assert out["deactivations"] == 60
        assert out["relaunches"] > 0          # at least one kernel was cut and resumed from its cursor


def test_two_queues_in_process_hpf_level2():
    hp, lp = run("--role", "both", "--kernel", "gemm", "--level", 2, "--count", 100, "--period-us", 5000, "--duration-s", 2,
                 "--hp-n", 1 << 24)
    assert hp["verified"] is True and hp["n"] >= 50
    assert lp["bit_exact"] is True and lp["iters"] > 10
    assert lp["deactivations"] > 10 and lp["relaunches"] > 0


def test_level1_window_only():
    hp, lp = run("--role", "both", "--kernel", "gemm", "--level", 1, "--count", 40, "--period-us", 10000, "--duration-s", 1,
                 "--hp-n", 1 << 24, "--M", 2048, "--N", 2048, "--K", 2048)
    assert hp["verified"] is True
    assert lp["bit_exact"] is True and lp["deactivations"] == 0
