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
