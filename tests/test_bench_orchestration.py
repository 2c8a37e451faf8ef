"""bench.py's process orchestration without a GPU: the helper that runs a high-priority process next to
long-running low-priority workers must open the workers' measurement window (SIGUSR1) when the HP process
reports READY, close it at DONE, and hand back the JSON lines; stand-in processes are small Python scripts."""
import importlib.util
import signal
import subprocess
import sys
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

FAKE_LP = r"""
import json, signal, sys, time
marks = []
signal.signal(signal.SIGUSR1, lambda *_: marks.append(time.time()))
stop = []
signal.signal(signal.SIGTERM, lambda *_: stop.append(1))
print("READY", flush=True)
while not stop:
    time.sleep(0.005)
print(json.dumps({"marks": marks}), flush=True)
"""

FAKE_HP = r"""
import json, sys, time
time.sleep(0.3)                 # start-up that must not count
print("READY", flush=True)
t0 = time.time()
time.sleep(0.4)                 # the requests
t1 = time.time()
print("DONE", flush=True)
time.sleep(0.3)                 # verification / tear-down that must not count
print(json.dumps({"t0": t0, "t1": t1}), flush=True)
"""


def load_bench():
    spec = importlib.util.spec_from_file_location("bench_module", ROOT / "bench.py")
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def test_lp_window_brackets_the_requests_only():
    bench = load_bench()
    lp = subprocess.Popen([sys.executable, "-c", FAKE_LP], stdout=subprocess.PIPE, text=True)
    assert lp.stdout.readline().startswith("READY")
    try:
        hp = bench.run_hp_marking([sys.executable, "-c", FAKE_HP], None, 30, [lp])[-1]
    finally:
        lp.send_signal(signal.SIGTERM)
        out, _ = lp.communicate(timeout=10)
    import json
    marks = json.loads(out.strip().splitlines()[-1])["marks"]
    assert len(marks) == 2
    assert abs(marks[0] - hp["t0"]) < 0.1 and abs(marks[1] - hp["t1"]) < 0.1
    assert 0.3 < marks[1] - marks[0] < 0.6


def test_failing_hp_process_is_reported_with_its_stderr():
    bench = load_bench()
    try:
        bench.run_hp_marking([sys.executable, "-c", "import sys; sys.stderr.write('boom'); sys.exit(3)"], None, 30, [])
    except RuntimeError as e:
        assert "rc=3" in str(e) and "boom" in str(e)
    else:
        raise AssertionError("no error raised")


# ---- the measurement method: percentiles over the timed requests only, on both sides --------------------------
FAKE_HP_WORKER = r"""#!/usr/bin/env python3
# Stand-in for the high-priority worker: `--count N --samples PATH`; the first requests are slow (a box that is
# still settling), the rest take 100 us with every fiftieth at 150 us.
import json, sys
a = dict(zip(sys.argv[1::2], sys.argv[2::2]))
n = int(a["--count"])
xs = [900.0 if i < 40 else (150.0 if i % 50 == 49 else 100.0) for i in range(n)]
open(a["--samples"], "w").write("\n".join(str(x) for x in xs))
s = sorted(xs)
print(json.dumps({"p50_us": s[len(s) // 2], "p99_us": s[int(0.99 * (len(s) - 1) + 0.5)], "xpk_launches": n, "argv_period": a.get("--period-us")}))
"""


def test_standalone_percentiles_ignore_the_untimed_requests(tmp_path):
    bench = load_bench()
    worker = tmp_path / "fake_worker"
    worker.write_text(FAKE_HP_WORKER)
    worker.chmod(0o755)
    bench.WORKER = worker
    r = bench.standalone_hp(0, None, 400, 50)
    assert len(r["samples_us"]) == 400                      # 450 requests were made, the first 50 are not timed
    assert r["p50_us"] == 100.0 and r["p99_us"] == 150.0    # the slow start is gone from both percentiles
    assert r["xpk_launches"] == 450
    # with no warm-up the worker's own figures would have carried the slow start into the P99
    r0 = bench.standalone_hp(0, None, 400, 0)
    assert r0["p99_us"] == 900.0
    # other workloads pass their own period and kernel through
    r3 = bench.standalone_hp(0, None, 100, 10, period_us=5000, hp_kernel="sort", hp_n=1 << 10)
    assert r3["argv_period"] == "5000" and len(r3["samples_us"]) == 100


def test_percentile_and_bootstrap_interval():
    bench = load_bench()
    xs = [float(i) for i in range(1, 101)]
    assert bench.pct(xs, 0.5) in (50.0, 51.0) and bench.pct(xs, 0.99) == 99.0 and bench.pct([7.0], 0.99) == 7.0
    co = [200.0 + (i % 10) for i in range(500)]
    alone = [100.0 + (i % 10) for i in range(500)]
    lo, hi = bench.ratio_interval(co, alone)
    point = bench.pct(co, 0.99) / bench.pct(alone, 0.99)
    assert lo - 1e-3 <= point <= hi + 1e-3 and 1.8 < lo and hi < 2.2        # the interval is rounded to four places
    assert bench.ratio_interval(co[:10], alone) is None     # too few samples for an interval


def test_mps_leg_reports_a_missing_control_binary(monkeypatch, tmp_path):
    bench = load_bench()
    monkeypatch.setenv("PATH", str(tmp_path))               # nothing named nvidia-cuda-mps-control here
    out = bench.mps_leg(0, "t.", {}, 10)
    assert "unavailable" in out and "nvidia-cuda-mps-control" in out["unavailable"]


def test_mps_leg_stops_the_daemon_when_a_worker_fails(monkeypatch, tmp_path):
    """A control binary that starts (exit 0 on -d) and records a `quit` on its standard input: whatever happens to
    the workers, the leg must send that quit."""
    bench = load_bench()
    log = tmp_path / "ctl.log"
    ctl = tmp_path / "nvidia-cuda-mps-control"
    ctl.write_text(f"#!/bin/sh\nif [ \"$1\" = \"-d\" ]; then echo started >> {log}; exit 0; fi\nread line; echo \"$line\" >> {log}\n")
    ctl.chmod(0o755)
    monkeypatch.setenv("PATH", f"{tmp_path}:/usr/bin:/bin")
    bad = tmp_path / "bad_worker"
    bad.write_text("#!/bin/sh\necho no gpu here >&2\nexit 5\n")
    bad.chmod(0o755)
    bench.WORKER = bad
    try:
        bench.mps_leg(0, "t.", {}, 10)
    except RuntimeError as e:
        assert "rc=5" in str(e)
    else:
        raise AssertionError("the failing worker went unnoticed")
    assert log.read_text().split() == ["started", "quit"]
