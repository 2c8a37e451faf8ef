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
