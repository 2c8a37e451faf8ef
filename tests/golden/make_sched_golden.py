"""Regenerate tests/golden/sched_scenarios_ref.json: the answers of the REFERENCE's LocalScheduler + HPF/LAX
(oracle/_ref/sched_probe_ref, compiled from the reference's sources by oracle/build_ref.py) on the scenarios
of tests/sched_scenarios.py.  Needs the reference tree at build time.

    python tests/golden/make_sched_golden.py
"""
import json
import sys
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tests"))

from sched_scenarios import SCENARIOS, run_probe  # noqa: E402

if __name__ == "__main__":
    out = {}
    for name, (policy, steps) in SCENARIOS.items():
        out[name] = [{str(pid): [list(r), list(s)] for pid, (r, s) in fl.items()} for fl in run_probe(ROOT / "oracle" / "_ref" / "sched_probe_ref", policy, steps)]
    (HERE / "sched_scenarios_ref.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {len(out)} scenarios")
