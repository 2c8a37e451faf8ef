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


def test_per_thread_default_stream_program_under_the_shim(shim_dir, tmp_path):
    """A program built with --default-stream per-thread: its two threads' default streams become two private
    streams with an XQueue each, and every launch and copy goes through them."""
    app = ROOT / "tests" / "apps" / "plain_ptds"
    assert app.exists(), "tests/apps/plain_ptds not built (python -m xsched_b200.build)"
    plain = subprocess.run([str(app), "25"], capture_output=True, text=True, timeout=120)
    assert plain.returncode == 0 and plain.stdout.startswith("OK"), plain.stdout + plain.stderr
    stats = tmp_path / "stats.json"
    r = subprocess.run([str(app), "25"], capture_output=True, text=True, timeout=180,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=1, XSCHED_AUTO_XQUEUE_THRESHOLD=4, XSCHED_AUTO_XQUEUE_BATCH_SIZE=2))
    assert r.returncode == 0, r.stdout + r.stderr[-2000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["thread_streams"] >= 2 and st["streams_with_xqueue"] >= 2
    assert st["launches_queued"] == 2 * 25 * 2          # two threads x rounds x two kernels
    assert st["copies_queued"] == 2 * 25 * 2
    assert st["getproc_hooked_ptsz"] > 0                 # the runtime asked for the per-thread variants and got the twins
    assert st["launches_direct"] == 0


def test_single_stream_per_process_mode(shim_dir, tmp_path):
    """XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS=ON: the program's two streams are one stream with one XQueue; the
    cross-stream event dependency of the test program still holds and the results are the same."""
    plain = subprocess.run([str(APP), "20"], capture_output=True, text=True, timeout=120)
    assert plain.returncode == 0
    stats = tmp_path / "stats.json"
    r = subprocess.run([str(APP), "20"], capture_output=True, text=True, timeout=180,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=1, XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS="ON"))
    assert r.returncode == 0, r.stdout + r.stderr[-2000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["streams_with_xqueue"] == 1 and st["single_stream_refs"] == 2
    assert st["launches_queued"] == 20 * 3


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


PAGEABLE_SCRIPT = r"""
import numpy as np, torch
s = torch.cuda.Stream()
total = 0
with torch.cuda.stream(s):
    dev = torch.empty(1 << 16, dtype=torch.int32, device="cuda")
    host = torch.empty(1 << 16, dtype=torch.int32)            # pageable
    for i in range(50):
        host.fill_(i)
        dev.copy_(host, non_blocking=True)                     # source may be reused as soon as the call returns
        host.fill_(-1)
        acc = (dev * 2).sum()
        out = torch.empty((), dtype=torch.int64)               # pageable destination
        out.copy_(acc, non_blocking=True)                      # readable as soon as the call returns
        total += int(out)
s.synchronize()
print(total)
"""


def test_pageable_copies_keep_their_synchronous_meaning(shim_dir, tmp_path):
    want = sum(2 * i * (1 << 16) for i in range(50))
    stats = tmp_path / "stats.json"
    r = subprocess.run([sys.executable, "-c", PAGEABLE_SCRIPT], capture_output=True, text=True, timeout=300,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=1))
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert int(r.stdout.strip()) == want
    st = json.loads(stats.read_text())
    assert st["copies_queued"] >= 100 and st["copies_waited"] >= 50, st


def test_library_kernels_are_queued_not_drained(shim_dir, tmp_path):
    # cuBLAS and the CUDA runtime launch library kernels (CUkernel handles); their arguments must be
    # copied like any other kernel's so that the stream's XQueue never drains for them.
    stats = tmp_path / "stats.json"
    r = subprocess.run([sys.executable, "-m", "xsched_b200.llama_decode", "--requests", "1", "--tokens", "4", "--rate", "50", "--layers", "2"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT, env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=1))
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    st = json.loads(stats.read_text())
    assert st["launches_queued"] > 200 and st["launches_blocking"] == 0, st


GRAPH_APP = ROOT / "tests" / "apps" / "plain_graph"


@pytest.mark.parametrize("level", [1, 2])
def test_graphs_and_other_stream_ordered_calls_under_the_shim(shim_dir, tmp_path, level):
    assert GRAPH_APP.exists(), "tests/apps/plain_graph not built (python -m xsched_b200.build)"
    plain = subprocess.run([str(GRAPH_APP), "20"], capture_output=True, text=True, timeout=120)
    assert plain.returncode == 0 and plain.stdout.startswith("OK"), plain.stdout + plain.stderr
    stats = tmp_path / "stats.json"
    r = subprocess.run([str(GRAPH_APP), "20"], capture_output=True, text=True, timeout=180,
                       env=shim_env(shim_dir, stats, XSCHED_AUTO_XQUEUE_LEVEL=level, XSCHED_AUTO_XQUEUE_THRESHOLD=4, XSCHED_AUTO_XQUEUE_BATCH_SIZE=2))
    assert r.returncode == 0, r.stdout + r.stderr[-2000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["graphs_queued"] == 40                    # two graph launches per round went through the XQueue
    # per round: memset2D, 2 graph launches, malloc/free async, memcpy2D, cooperative launch, stream callback (+ one upload)
    assert st["calls_queued"] >= 20 * 8, st
    assert st["launches_queued"] == 20 * 2              # captured launches bypass the XQueue; add_one + times_two per round do not
