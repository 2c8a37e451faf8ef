"""Regenerate tests/golden/host_*.json from the reference's own host core.

Runs oracle/_ref/lane_driver_ref (the scenario runner linked against the reference core compiled by
oracle/build_ref.py — that needs the reference tree) and stores what it prints.  Only the
timing-independent fields are compared by the tests; the rest is kept for information.

    python tests/golden/make_host_golden.py
"""
import json
import os
import subprocess
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
DRIVER = ROOT / "oracle" / "_ref" / "lane_driver_ref"

SCENARIOS = {
    "api_contract": ["api_contract"],
    "window_4_2": ["window", "4", "2", "40", "300"],
    "window_16_8": ["window", "16", "8", "100", "200"],
    "window_1_1": ["window", "1", "1", "12", "300"],
    "suspend_l1": ["suspend", "1", "40", "500"],
    "suspend_l2": ["suspend", "2", "40", "500"],
    "drop_l1": ["drop", "1", "40", "500"],
    "drop_l2": ["drop", "2", "40", "500"],
    # seeded random walks over the C API (result codes, counters and quiescent states only)
    "fuzz_seed_1": ["fuzz", "1", "200"],
    "fuzz_seed_2": ["fuzz", "2", "200"],
    "fuzz_seed_3": ["fuzz", "3", "200"],
    "fuzz_seed_11": ["fuzz", "11", "300"],
}


def main() -> None:
    env = dict(os.environ, XLOG_LEVEL="ERRO")
    out = {}
    for name, args in SCENARIOS.items():
        r = subprocess.run([str(DRIVER), *args], capture_output=True, text=True, env=env, timeout=120, check=True)
        out[name] = {"args": args, "result": json.loads(r.stdout)}
    (HERE / "host_scenarios_ref.json").write_text(json.dumps(out, indent=1, sort_keys=True) + "\n")
    print(f"wrote {HERE / 'host_scenarios_ref.json'} ({len(out)} scenarios)")


if __name__ == "__main__":
    main()
