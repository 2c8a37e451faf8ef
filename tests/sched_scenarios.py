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
    # ---- the other policies.  Sleeps sit at least 100 ms away from every slice boundary. ----
    "hhpf_one_maximum_over_all_devices": ("HHPF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV2),
        ("ev", "hint_priority", P2, B, 5),
        ("ev", "xq_ready", P1, A, 0.0), ("flush",),
        ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("ev", "xq_idle", P2, B), ("flush",),
    ]),
    "up_turns_by_utilization": ("UP", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "proc_create", P3),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1), ("ev", "xq_create", P3, C, DEV1),
        ("ev", "hint_timeslice", P1, 800_000), ("ev", "hint_utilization", P1, P1, A, 75), ("ev", "hint_utilization", P2, P2, B, 25),
        ("ev", "xq_ready", P3, C, 0.0), ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("flush",),   # A: 600 ms
        ("sleep_ms", 300), ("flush",),                # still A
        ("sleep_ms", 400), ("flush",),                # t = 700: B's 200 ms turn (600..800)
        ("sleep_ms", 250), ("flush",),                # t = 950: A again (800..1400)
        ("ev", "xq_idle", P1, A), ("flush",),         # the holder went idle: B takes over at once
    ]),
    "pup_turns_by_process": ("PUP", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P1, B, DEV1), ("ev", "xq_create", P2, C, DEV1),
        ("ev", "hint_timeslice", P1, 300_000), ("ev", "hint_utilization", P1, P1, 0, 50), ("ev", "hint_utilization", P2, P2, 0, 50),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, C, 0.0), ("flush",),    # P1 runs 300 ms
        ("sleep_ms", 150), ("flush",),
        ("sleep_ms", 300), ("flush",),                # t = 450: P2's turn (300..600)
        ("ev", "xq_idle", P2, C), ("flush",),         # P2 idle with time left: P1 gets the GPU back
    ]),
    "kedf_k_earliest": ("KEDF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "proc_create", P3),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1), ("ev", "xq_create", P3, C, DEV1),
        ("ev", "hint_deadline", P1, A, 50_000_000), ("ev", "hint_deadline", P2, B, 20_000_000),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("ev", "xq_ready", P3, C, 0.0), ("flush",),   # B alone
        ("ev", "hint_kdeadline", P1, 2), ("flush",),                                                                # B and A
        ("ev", "xq_idle", P2, B), ("flush",),                                                                       # A and (never) B or C
        ("ev", "hint_kdeadline", P1, 0), ("ev", "hint_kdeadline", P1, 1), ("flush",),
    ]),
    "awf_active_window": ("AWF", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1),
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P2, B, 0.0), ("flush",),
        ("ev", "hint_window_active", P1, P2, 7), ("flush",),          # P2 owns the active window: P1 waits
        ("ev", "hint_window_active", P1, P1, 7), ("flush",),          # focus moves on the same display
        ("ev", "xq_idle", P1, A), ("flush",),                         # the active process is idle: everybody runs
        ("ev", "hint_window_active", P1, 0, 7), ("flush",),           # pid 0 is ignored
    ]),
    "cfs_catch_up": ("CFS", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "proc_create", P3),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1), ("ev", "xq_create", P3, C, DEV2),
        ("ev", "hint_priority", P2, B, 0),                            # B is known (virtual runtime 0) before it ever runs
        ("ev", "xq_ready", P1, A, 0.0), ("ev", "xq_ready", P3, C, 0.0), ("flush",),
        ("sleep_ms", 500), ("flush",),                                # A has run 500 ms alone on its device
        ("ev", "xq_ready", P2, B, 0.0), ("flush",),                   # B is far behind: it runs, A waits
        ("sleep_ms", 250), ("flush",),                                # still catching up
    ]),
    "mlfq_levels": ("MLFQ", [
        ("ev", "proc_create", P1), ("ev", "proc_create", P2), ("ev", "proc_create", P3),
        ("ev", "xq_create", P1, A, DEV1), ("ev", "xq_create", P2, B, DEV1), ("ev", "xq_create", P3, C, DEV1),
        ("ev", "xq_ready", P1, A, 0.0), ("flush",),
        ("sleep_ms", 300), ("flush",),                                # A alone sank to the lowest level but keeps running
        ("ev", "xq_ready", P2, B, 0.0), ("flush",),                   # B (level 0) takes over for its first 70 ms
        ("ev", "xq_idle", P2, B), ("flush",),                         # and A gets the device back when B is done
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
        elif st[0] in ("flush", "peek"):
            lines.append(st[0])
        elif st[0] == "sleep_us":
            lines.append(f"sleep_us {st[1]}")
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


def run_virtual(binary, policy, steps, t0_us: int, env_extra=None):
    """The product's scheduler on a virtual clock starting at t0_us (exactly reproducible)."""
    env = dict(os.environ, XLOG_LEVEL="ERRO")
    env.update(env_extra or {})
    r = subprocess.run([str(binary), policy, "--virtual", str(t0_us)], input=script_text(steps, t0_us), capture_output=True, text=True, env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-1000:]
    return parse_flushes(r.stdout)


def random_steps(policy: str, seed: int, n: int = 400):
    """A seeded random walk over events, hints and short sleeps (virtual-clock comparisons only)."""
    import random
    rng = random.Random(seed)
    pids = [P1, P2, P3]
    queues = {A: (P1, DEV1), B: (P2, DEV1), C: (P3, DEV1), D: (P3, DEV2), 0xE5: (P1, DEV2)}
    steps = [("ev", "proc_create", p) for p in pids]
    steps += [("ev", "xq_create", pid, h, dev) for h, (pid, dev) in queues.items()]
    ready = {h: False for h in queues}
    for _ in range(n):
        x = rng.random()
        h = rng.choice(list(queues))
        pid = queues[h][0]
        if x < 0.30:
            ready[h] = not ready[h]
            steps.append(("ev", "xq_ready", pid, h, 0.0) if ready[h] else ("ev", "xq_idle", pid, h))
        elif x < 0.40:
            steps.append({
                "HPF": ("ev", "hint_priority", pid, h, rng.randint(-3, 3)), "HHPF": ("ev", "hint_priority", pid, h, rng.randint(-3, 3)),
                "CFS": ("ev", "hint_priority", pid, h, rng.randint(-3, 3)),
                "LAX": ("ev", "hint_laxity", pid, h, rng.choice([-1, 2000, 20000]), rng.randint(-2, 2), rng.randint(-2, 4)),
                # (no zero shares: a zero budget makes the reference's timer fire in a tight loop)
                "UP": ("ev", "hint_utilization", pid, pid, h, rng.choice([-1, 10, 30, 60, 100, 101])),
                "PUP": ("ev", "hint_utilization", pid, rng.choice(pids + [0]), 0, rng.choice([-1, 10, 30, 60, 100, 101])),
                "KEDF": rng.choice([("ev", "hint_deadline", pid, h, rng.choice([1000, 5000, 50000])), ("ev", "hint_kdeadline", pid, rng.randint(0, 3))]),
                "AWF": ("ev", "hint_window_active", pid, rng.choice(pids + [0]), rng.randint(1, 2)),
                "MLFQ": ("ev", "hint_priority", pid, h, 1),
            }[policy])
        elif x < 0.45 and policy in ("UP", "PUP"):
            steps.append(("ev", "hint_timeslice", pid, rng.choice([3000, 20000, 20_000_000] + ([50] if policy == "PUP" else []))))   # 50: refused by PUP
        elif x < 0.85:
            steps.append(("sleep_ms", rng.choice([1, 2, 3, 7, 12, 40, 90])))
        else:
            steps.append(("flush",))
    steps.append(("flush",))
    return steps


def run_model(policy, steps, scope="GLOBAL", t0_us: int | None = None):
    """The Python restatement, stepping a virtual clock across sleeps."""
    m = so.Model(policy, scope)
    t0 = so.now_us() if t0_us is None else t0_us
    now = t0
    out = []
    for st in steps:
        if st[0] == "ev":
            m.apply(build_event(st, t0))
            m.decide(now)                  # a round after every event: the no-batching extreme
        elif st[0] == "sleep_ms":
            now = m.advance(now, now + st[1] * 1000)
        else:
            now = m.advance(now, now + 30_000)      # the probes let 30 ms pass before they report
            out.append(m.snapshot())
    return out
