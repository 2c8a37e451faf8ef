"""Scheduling parity: this repository's LocalScheduler + HPF/LAX against (1) the reference's own
LocalScheduler and policies compiled from its sources (live when present, committed golden answers always)
and (2) the pure-Python restatement in oracle/sched_oracle.py.  The same raw event bytes go to all three,
so the test also pins the record layouts."""
import json
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
sys.path.insert(0, str(ROOT / "tests"))
from sched_scenarios import SCENARIOS, run_model, run_probe  # noqa: E402

NEW = ROOT / "oracle" / "sched_probe_new"
REF = ROOT / "oracle" / "_ref" / "sched_probe_ref"
GOLDEN = json.loads((ROOT / "tests" / "golden" / "sched_scenarios_ref.json").read_text())


def norm(flushes):
    return [{int(pid): (tuple(sorted(r)), tuple(sorted(s))) for pid, (r, s) in fl.items()} for fl in flushes]


@pytest.fixture(scope="module", autouse=True)
def built():
    if not NEW.exists():
        from xsched_b200 import build
        build.build_host()
        build.build_lane_driver()
    assert NEW.exists()


@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_matches_reference_golden_and_python_restatement(name):
    policy, steps = SCENARIOS[name]
    got = norm(run_probe(NEW, policy, steps))
    golden = norm([{int(p): (v[0], v[1]) for p, v in fl.items()} for fl in GOLDEN[name]])
    model = norm(run_model(policy, steps))
    assert got == golden, f"product differs from the reference's answers on {name}"
    assert model == golden, f"python restatement differs from the reference's answers on {name}"


@pytest.mark.skipif(not REF.exists(), reason="compiled reference core not present")
@pytest.mark.parametrize("name", sorted(SCENARIOS))
def test_matches_live_reference(name):
    policy, steps = SCENARIOS[name]
    assert norm(run_probe(NEW, policy, steps)) == norm(run_probe(REF, policy, steps))


def test_lax_device_scope_is_independent_per_gpu():
    """XSCHED_POLICY_SCOPE=DEVICE (an addition): a critical queue on one GPU does not suspend queues on another."""
    policy, steps = SCENARIOS["lax_global_scope_across_devices"]
    glob = norm(run_probe(NEW, policy, steps))
    dev = norm(run_probe(NEW, policy, steps, env_extra={"XSCHED_POLICY_SCOPE": "DEVICE"}))
    assert glob[-1][100] == ((), (0xA1,))            # reference behaviour: suspended by the other device's queue
    assert dev[-1][100] == ((0xA1,), ())
    assert norm(run_model(policy, steps, scope="DEVICE")) == dev


VIRTUAL_T0 = 1_800_000_000_000_000


@pytest.mark.parametrize("policy", ["HPF", "HHPF", "LAX", "UP", "PUP", "KEDF", "AWF", "CFS", "MLFQ"])
def test_random_walks_on_a_virtual_clock_match_the_python_restatement(policy):
    """Seeded random event/hint/sleep sequences, the product's scheduler stepping a virtual clock: every
    report must equal the Python restatement's, millisecond-scale slice and tick effects included (the
    real-time scenarios above can only probe outcomes that hold for >= 100 ms)."""
    from sched_scenarios import random_steps, run_virtual
    for seed in range(4):
        steps = random_steps(policy, seed, n=300)
        got = norm(run_virtual(NEW, policy, steps, VIRTUAL_T0))
        want = norm(run_model(policy, steps, t0_us=VIRTUAL_T0))
        assert got == want, f"{policy} seed {seed}: first difference at report {next(i for i, (a, b) in enumerate(zip(got, want)) if a != b)}"


def test_chpf_follows_linux_priorities():
    """CHPF reads /proc/<pid>/sched: a reniced process ranks below a normal one.  Real processes are needed,
    so the answer cannot be committed as a golden file: product, Python restatement and (when built) the
    compiled reference are compared live."""
    import os
    import subprocess
    from oracle import sched_oracle as so
    normal = subprocess.Popen(["sleep", "60"])
    nicer = subprocess.Popen(["nice", "-n", "10", "sleep", "60"])
    try:
        import time
        time.sleep(0.2)
        assert so.linux_priority(normal.pid) > so.linux_priority(nicer.pid)
        A, B, DEV = 0xA1, 0xB2, (2 << 32) | 0x1000
        steps = [("ev", "proc_create", normal.pid), ("ev", "proc_create", nicer.pid),
                 ("ev", "xq_create", normal.pid, A, DEV), ("ev", "xq_create", nicer.pid, B, DEV),
                 ("ev", "hint_priority", nicer.pid, B, 200),             # hints are ignored by this policy
                 ("ev", "xq_ready", nicer.pid, B, 0.0), ("flush",),
                 ("ev", "xq_ready", normal.pid, A, 0.0), ("flush",),
                 ("ev", "xq_idle", normal.pid, A), ("flush",)]
        got = norm(run_probe(NEW, "CHPF", steps))
        assert got == norm(run_model("CHPF", steps))
        assert got[1][nicer.pid] == ((), (B,)) and got[2][nicer.pid] == ((B,), ())
        if REF.exists():
            assert got == norm(run_probe(REF, "CHPF", steps))
    finally:
        normal.kill(); nicer.kill()
        normal.wait(); nicer.wait()


def test_hpf_resume_hysteresis_keeps_lower_priorities_out_of_short_gaps():
    """XSCHED_HPF_RESUME_HYSTERESIS_US (an addition; off by default): a high-priority queue that goes idle and comes
    back within the window never lets the low-priority queue be resumed in between; once the window has passed
    the low-priority queue runs again.  Without the variable every idle edge resumes at once, as in the reference."""
    from sched_scenarios import run_virtual, A, B, P1, P2, DEV1
    steps = [("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1),
             ("ev", "hint_priority", P2, B, 1), ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("peek",),      # 0: A suspended
             ("ev", "xq_idle", P2, B), ("peek",),                                                                                  # 1: the gap
             ("sleep_us", 300), ("ev", "xq_ready", P2, B, 0.0), ("peek",),                                                         # 2: B back within the window
             ("ev", "xq_idle", P2, B), ("sleep_us", 999), ("peek",),                                                                # 3: window not yet over
             ("sleep_us", 2), ("peek",)]                                                                                            # 4: over
    run, susp = ((A,), ()), ((), (A,))
    with_h = [f[P1] for f in run_virtual(NEW, "HPF", steps, VIRTUAL_T0, env_extra={"XSCHED_HPF_RESUME_HYSTERESIS_US": "1000"})]
    assert with_h == [susp, susp, susp, susp, run]
    plain = [f[P1] for f in run_virtual(NEW, "HPF", steps, VIRTUAL_T0)]
    assert plain == [susp, run, susp, run, run]
