"""Scripted event sequences for the scheduler parity tests (shared with tests/golden/make_sched_golden.py).

A step is ("ev", builder_name, args...) | ("flush",) | ("sleep_ms", n).  Times in ready events are
offsets from "now" in seconds, large enough (>= 5 s either way) that the outcome cannot depend on how
fast the probe runs — except the timer scenario, which sleeps across a 300 ms laxity on purpose.
"""
from __future__ import annotations

import os
import subprocess

from oracle import sched_oracle as so

A, B, C, D = 0xA1, 0xB2, 0xC3, 0xD4
P1, P2, P3 = 100, 200, 300
DEV1, DEV2 = (2 << 32) | 0x1000, (2 << 32) | 0x2000

SCENARIOS = {
    "hpf_basic": ("HPF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1),
        ("ev", "hint_priority", P1, A, 0), ("ev", "hint_priority", P2, B, 1),
        ("ev", "xq_ready", P1, A, 0.0), ("flush",),
        ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("ev", "xq_idle", P2, B), ("flush",),
        ("ev", "xq_ready", P2, B, 0.0), ("ev", "xq_idle", P1, A), ("flush",),
    ]),
    "hpf_per_device": ("HPF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "proc_create", P3),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV2), ("ev", "xq_create", P3, C, DEV1), ("ev", "xq_create", P3, D, DEV2),
        ("ev", "hint_priority", P2, B, 5), ("ev", "hint_priority", P3, C, 3), ("ev", "hint_priority", P3, D, -7),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("ev", "xq_ready", P3, C, 0.0), ("flush",),
        ("ev", "xq_ready", P3, D, 0.0), ("flush",),
        ("ev", "xq_idle", P2, B), ("flush",),
    ]),
    "hpf_clamp_default_equal": ("HPF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P1, B, DEV1), ("ev", "xq_create", P2, C, DEV1),
        ("ev", "hint_priority", P1, A, 999), ("ev", "hint_priority", P2, C, 255),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P1, B, 0.0), ("ev", "xq_ready", P2, C, 0.0), ("flush",),
        ("ev", "hint_priority", P1, B, -999), ("ev", "xq_idle", P1, A), ("ev", "xq_idle", P2, C), ("flush",),
    ]),
    "hpf_process_and_queue_destroy": ("HPF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1), ("ev", "xq_create", P2, C, DEV1),
        ("ev", "hint_priority", P2, B, 2), ("ev", "hint_priority", P2, C, 1),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("ev", "xq_ready", P2, C, 0.0), ("flush",),
        ("ev", "xq_destroy", P2, B), ("flush",),
        ("ev", "proc_destroy", P2), ("flush",),
    ]),
    "hpf_ready_for_unknown_queue": ("HPF", [
        ("ev", "proc_create", P1),
        ("ev", "xq_ready", P1, A, 0.0), ("flush",),
        ("ev", "xq_create", P1, B, DEV1, True), ("ev", "hint_priority", P1, B, 4), ("ev", "xq_ready", P1, B, 0.0), ("flush",),
    ]),
    "lax_relaxed_then_critical": ("LAX", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1),
        ("ev", "hint_laxity", P2, B, 10_000_000, -5, 7),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("ev", "xq_idle", P2, B), ("ev", "xq_ready", P2, B, -20.0), ("flush",),
        ("ev", "xq_idle", P1, A), ("flush",),
    ]),
    "lax_global_scope_across_devices": ("LAX", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV2),
        ("ev", "hint_laxity", P2, B, 1_000_000, 0, 9),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, -30.0), ("flush",),
    ]),
    "lax_timer_flip": ("LAX", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1),
        ("ev", "hint_laxity", P2, B, 300_000, -5, 7),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("sleep_ms", 600), ("flush",),
    ]),
}


def build_event(step, t0_us: int) -> bytes:
    name, args = step[1], list(step[2:])
    if name == "xq_ready":
        args[2] = t0_us + int(args[2] * 1e6)
    if name == "xq_create" and len(args) == 4:
        return so.ev_xq_create(args[0], args[1], args[2], update=bool(args[3]))
    return getattr(so, "ev_" + name)(*args)


def script_text(steps, t0_us: int) -> str:
    lines = []
    for st in steps:
        if st[0] == "ev":
            lines.append("event " + build_event(st, t0_us).hex())
        elif st[0] == "flush":
            lines.append("flush")
        else:
            lines.append(f"sleep_ms {st[1]}")
    return "\n".join(lines) + "\n"


def parse_flushes(text: str):
    out = []
    for line in text.splitlines():
        if not line.startswith("flush"):
            continue
        d = {}
        for part in line.split("|")[1:]:
            tok = part.split()
            pid = int(tok[1])
            i_run, i_susp = tok.index("run"), tok.index("susp")
            d[pid] = (tuple(int(x, 16) for x in tok[i_run + 1:i_susp]), tuple(int(x, 16) for x in tok[i_susp + 1:]))
        out.append(d)
    return out


def run_probe(binary, policy, steps, env_extra=None):
    env = dict(os.environ, XLOG_LEVEL="ERRO")
    env.update(env_extra or {})
    r = subprocess.run([str(binary), policy], input=script_text(steps, so.now_us()), capture_output=True, text=True, env=env, timeout=60)
    assert r.returncode == 0, r.stderr[-1000:]
    return parse_flushes(r.stdout)


def run_model(policy, steps, scope="GLOBAL"):
    """The Python restatement, stepping a virtual clock across sleeps."""
    m = so.Model(policy, scope)
    t0 = so.now_us()
    now = t0
    out = []
    for st in steps:
        if st[0] == "ev":
            m.apply(build_event(st, t0))
        elif st[0] == "sleep_ms":
            now += st[1] * 1000
        else:
            out.append(m.decide(now))
    return out
