"""Host runtime (XQueue C API, window, suspend/resume, drop, HPF) against the reference's own core.

The same scenario runner (oracle/lane_driver.cpp, C API only) is built against both code bases.  The
timing-independent fields must be identical to the committed golden output of the reference
(tests/golden/host_scenarios_ref.json) and, when the compiled reference core is present, to a live
run of it.  Timing-dependent fields are checked against bounds that follow from the algorithm.
"""
import json
import os
import subprocess
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
NEW = ROOT / "oracle" / "lane_driver_new"
REF = ROOT / "oracle" / "_ref" / "lane_driver_ref"
GOLDEN = json.loads((ROOT / "tests" / "golden" / "host_scenarios_ref.json").read_text())
TIMING_KEYS = {"suspend_us", "suspend_bound_us", "flushed_any", "partial_at_suspend"}
# Some fields are decided by the algorithm on an idle host but can come out differently when the host is so busy
# that the lane thread or the submitting thread loses its core for milliseconds (was anything still queued at the
# moment of the suspension?  was the queue still ready right after the submissions?), and latency bounds assume
# that a 1 ms busy-spin takes about 1 ms.  Such checks run in up to three attempts: an attempt that matches proves
# the behaviour, a loaded host only makes an attempt inconclusive.


def eventually(check, attempts=3):
    """Run `check` (which asserts) until it passes, at most `attempts` times; the last failure is raised."""
    for i in range(attempts):
        try:
            return check()
        except AssertionError:
            if i == attempts - 1:
                raise


def run(driver, args, timeout=180):
    env = dict(os.environ, XLOG_LEVEL="ERRO")
    r = subprocess.run([str(driver), *map(str, args)], capture_output=True, text=True, env=env, timeout=timeout)
    assert r.returncode == 0, r.stderr[-2000:]
    return json.loads(r.stdout)


@pytest.fixture(scope="module", autouse=True)
def built():
    if not NEW.exists():
        from xsched_b200 import build
        build.build_host()
        build.build_lane_driver()
    assert NEW.exists()


def strip(d):
    return {k: v for k, v in d.items() if k not in TIMING_KEYS}


@pytest.mark.parametrize("name", sorted(GOLDEN))
def test_scenario_matches_reference_golden(name):
    want = GOLDEN[name]["result"]

    def check():
        got = run(NEW, GOLDEN[name]["args"])
        if name == "api_contract":
            # Asking for the local scheduler with kPolicyUnknown while application-managed: both accept.
            assert got == want
        else:
            assert strip(got) == strip(want)
        if "suspend_us" in got:
            assert got["suspend_us"] <= got["suspend_bound_us"], got
            # whether commands were still queued when the suspension came depends on the host keeping time
            assert (got["flushed_any"], got["partial_at_suspend"]) == (want["flushed_any"], want["partial_at_suspend"]), got
    eventually(check, attempts=5)


@pytest.mark.skipif(not REF.exists(), reason="compiled reference core not present")
@pytest.mark.parametrize("name", ["api_contract", "window_4_2", "suspend_l2", "drop_l2", "fuzz_seed_11"])
def test_scenario_matches_live_reference(name):
    args = GOLDEN[name]["args"]

    def check():
        assert strip(run(NEW, args)) == strip(run(REF, args))
    eventually(check)


def _hpf(driver, level):
    return run(driver, ["hpf", level, 300, 1000, 8, 2000, 30000, 16, 8])


def test_hpf_level1_latency_is_window_bound_and_level2_is_not():
    eventually(_check_hpf_shape)


def _check_hpf_shape():
    l1, l2 = _hpf(NEW, 1), _hpf(NEW, 2)
    # Level 1: the high-priority command waits for the in-flight window (<= 16 x 1 ms) to drain.
    assert l1["hp"]["p50_us"] > 6000
    # Level 2: not-yet-started commands are pulled back; at most the running one (1 ms) is in the way.  The median
    # is held against the algorithmic figure with slack for a busy host, and against level 1 on the same host.
    assert l2["hp"]["p50_us"] <= 2000 + 1000 + 7000
    assert l2["hp"]["p50_us"] < 0.6 * l1["hp"]["p50_us"]
    assert l2["flushed"] > 0
    # the low-priority work still completes, in about its own time plus the high-priority work
    for r in (l1, l2):
        assert r["hp"]["lp_total_ms"] <= (300 * 1.0 + 8 * 2.0) * 2.0 + 50


@pytest.mark.skipif(not REF.exists(), reason="compiled reference core not present")
def test_hpf_same_behaviour_as_reference_core():
    def check():
        for level in (1, 2):
            a, b = _hpf(NEW, level), _hpf(REF, level)
            assert abs(a["hp"]["p50_us"] - b["hp"]["p50_us"]) <= 0.5 * b["hp"]["p50_us"] + 3000
            assert abs(a["hp"]["lp_total_ms"] - b["hp"]["lp_total_ms"]) <= 0.1 * b["hp"]["lp_total_ms"] + 10
    eventually(check)


def _lax(driver, level, lax_us=5000):
    return run(driver, ["lax", level, 300, 1000, 6, 2000, 40000, 16, 8, "LCL", lax_us])


def test_lax_high_priority_waits_its_laxity_then_preempts():
    eventually(_check_lax_shape)


def _check_lax_shape():
    # Laxity policy on the host lane at level 2: the hinted queue is relaxed (priority 0, served in FIFO
    # order behind up to 16 x 1 ms commands) for 5 ms after it becomes ready, then critical: the other
    # queue is deactivated, at most the running 1 ms command is in the way, then its own 2 ms run.
    r = _lax(NEW, 2)
    assert 5000 + 2000 <= r["hp"]["p50_us"] <= 5000 + 1000 + 2000 + 6000, r
    assert r["flushed"] > 0
    # a laxity longer than the window's natural drain never turns critical: same as level 1, no flush
    slack = _lax(NEW, 2, 60000)
    assert slack["flushed"] == 0 and slack["hp"]["p50_us"] > 8000, slack


@pytest.mark.skipif(not REF.exists(), reason="compiled reference core not present")
def test_lax_same_behaviour_as_reference_core():
    def check():
        a, b = _lax(NEW, 2), _lax(REF, 2)
        assert abs(a["hp"]["p50_us"] - b["hp"]["p50_us"]) <= 4000, (a, b)
        assert (a["flushed"] > 0) == (b["flushed"] > 0)
    eventually(check)


def test_lax_through_the_server_per_device():
    # The same scenario with the policy in an xserver (laxity policy, per-device scope).
    import os
    import signal
    import subprocess
    ns = f"lax{os.getpid()}."
    env = dict(os.environ, XLOG_LEVEL="WARN", XSCHED_IPC_NAMESPACE=ns, XSCHED_POLICY_SCOPE="DEVICE")
    env.pop("XSCHED_SCHEDULER", None)
    srv = subprocess.Popen([str(NEW.parent.parent / "xsched_b200" / "lib" / "xserver"), "LAX", "50000"], stdout=subprocess.PIPE, text=True, env=env)
    try:
        assert "ready" in srv.stdout.readline()
        out = subprocess.run([str(NEW), "lax", "2", "300", "1000", "6", "2000", "40000", "16", "8", "GLB", "5000"], capture_output=True, text=True,
                             env=dict(env, XLOG_LEVEL="ERRO"), timeout=120)
        assert out.returncode == 0, out.stderr[-800:]
        import json
        r = json.loads(out.stdout.strip().splitlines()[-1])
        assert 5000 + 2000 <= r["hp"]["p50_us"] <= 5000 + 1000 + 2000 + 8000, r
        assert r["flushed"] > 0
    finally:
        srv.send_signal(signal.SIGTERM)
        srv.wait(timeout=10)


@pytest.mark.skipif(not REF.exists(), reason="compiled reference core not present")
def test_random_api_walks_match_the_live_reference():
    """Fresh seeds every run of the suite would make failures irreproducible; a fixed block of seeds beyond the
    committed golden ones is walked instead.  Result codes, counters and quiescent states must be identical and
    every command that was not dropped must have run exactly once, in both implementations."""
    for seed in range(100, 112):
        a, b = run(NEW, ["fuzz", seed, 200]), run(REF, ["fuzz", seed, 200])
        assert a == b, f"seed {seed}"
        assert a["all_ran_unless_dropped"] == 1 and a["none_ran_twice"] == 1, f"seed {seed}"


def test_manual_suspend_resume_next_to_a_scheduler_never_strands_commands():
    """An application suspends and resumes its XQueue by hand while the in-process scheduler manages the same
    queue (its first operation for a new queue is a Resume, executed on the agent's thread).  Suspend and
    Resume are serialised, so whatever order the two threads arrive in, every command runs exactly once and
    XQueueWaitAll returns.  The window is widest right after process start: many short-lived processes."""
    from concurrent.futures import ThreadPoolExecutor

    def one(_):
        r = subprocess.run([str(NEW), "stress", "2", "1", "500"], capture_output=True, text=True, env=dict(os.environ, XLOG_LEVEL="ERRO"), timeout=60)
        return r.returncode, r.stdout
    with ThreadPoolExecutor(max_workers=12) as pool:
        for rc, out in pool.map(one, range(60)):
            assert rc == 0, out
            res = json.loads(out)
            assert res["executed"] == res["expected"], res
    res = run(NEW, ["stress", 2, 400, 100])
    assert res["executed"] == res["expected"] == 2400


@pytest.mark.parametrize("level", [1, 2])
def test_concurrent_submit_suspend_query_loses_nothing(level):
    """Three threads on one XQueue — one submits bursts and waits, one suspends/resumes at random (with and
    without SyncHwQueue), one queries, counts and hints — next to the in-process scheduler.  Nothing is dropped,
    so every command must run exactly once and every wait must return.  (The reference core, driven by the same
    scenario at level 2, strands a few commands in about one run out of six; nothing is asserted about it.)"""
    for seed in (1, 2, 3):
        res = run(NEW, ["mtfuzz", seed, level, 200])
        assert res["submitted"] == res["executed"], (seed, res)
