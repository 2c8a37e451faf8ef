"""The libcuda interposer on a GPU: an XSched-unaware CUDA program and a PyTorch script run unchanged under
LD_LIBRARY_PATH=<shim dir>, produce the same results, and their stream work demonstrably went through XQueues."""
import json
import os
import subprocess
import sys
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
APP = ROOT / "tests" / "apps" / "plain_streams"


@pytest.fixture(scope="module")
def shim_dir(tmp_path_factory):
    d = tmp_path_factory.mktemp("shim")
    for name in ("libcuda.so.1", "libcuda.so"):
        os.symlink(LIB / "libshimcuda.so", d / name)
    return d


def shim_env(shim_dir, stats, **extra):
    env = dict(os.environ, XLOG_LEVEL="WARN", XSCHED_AUTO_XQUEUE="ON", XSCHED_POLICY="HPF", XSCHED_SHIM_STATS_FILE=str(stats))
    env["LD_LIBRARY_PATH"] = f"{shim_dir}:{LIB}:" + env.get("LD_LIBRARY_PATH", "")
    env.pop("XSCHED_SCHEDULER", None)
    env.update({k: str(v) for k, v in extra.items()})
    return env


@pytest.mark.parametrize("level", [1, 2])
def test_plain_cuda_program_under_the_shim(shim_dir, tmp_path, level):
    assert APP.exists(), "tests/apps/plain_streams not built (python -m xsched_b200.build)"
    plain = subprocess.run([str(APP), "40"], capture_output=True, text=True, timeout=120)
    assert plain.returncode == 0 and plain.stdout.startswith("OK"), plain.stdout + plain.stderr
    stats = tmp_path / "stats.json"
    r = subprocess.run([str(APP), "40"], capture_output=True, text=True, timeout=180,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=level, XSCHED_AUTO_XQUEUE_THRESHOLD=4, XSCHED_AUTO_XQUEUE_BATCH_SIZE=2))
    assert r.returncode == 0, r.stdout + r.stderr[-2000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["streams_with_xqueue"] == 2
    assert st["launches_queued"] == 40 * 3              # two vector_add + one scale per round
    assert st["copies_queued"] == 40 * 6
    assert st["events_queued"] == 40
    assert st["syncs_via_xqueue"] >= 80
    assert st["getproc_hooked"] > 0                     # the runtime resolved its entry points through the override


TORCH_SCRIPT = r"""
import torch
torch.manual_seed(0)
s = torch.cuda.Stream()
with torch.cuda.stream(s):
    a = torch.randn(1024, 1024, device="cuda")
    b = a @ a
    for _ in range(20):
        b = torch.relu(b @ a) * 1e-3
    c = b.float().sum()
s.synchronize()
print("%.6e" % float(c))
"""


def test_pytorch_under_the_shim_gives_the_same_numbers(shim_dir, tmp_path):
    plain = subprocess.run([sys.executable, "-c", TORCH_SCRIPT], capture_output=True, text=True, timeout=300)
    assert plain.returncode == 0, plain.stderr[-2000:]
    stats = tmp_path / "stats.json"
    r = subprocess.run([sys.executable, "-c", TORCH_SCRIPT], capture_output=True, text=True, timeout=300,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=1))
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert r.stdout.strip() == plain.stdout.strip()
    st = json.loads(stats.read_text())
    assert st["streams_with_xqueue"] >= 1 and st["launches_queued"] >= 40
