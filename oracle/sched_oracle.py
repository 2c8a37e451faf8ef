"""Pure-Python restatement of the scheduling half of the path (TEST INFRASTRUCTURE).

* record layouts of the agent -> server events and hints, as the reference defines them:
    EventMeta {int32 type; int32 pid}                      sched/include/xsched/sched/protocol/event.h:33-37
    XQueueCreate/ConfigUpdate {meta, handle, device, level, threshold, batch}   event.h:146-205, :290-349
    XQueueDestroy/Idle {meta, handle}; XQueueReady {meta, handle, ready_time_us}  event.h:207-288
    ProcessCreate {meta, char cmdline[256]}; ProcessDestroy {meta}               event.h:101-143
    HintEvent {meta, size_t size, hint bytes}                                    event.h:55-84
    PriorityHint {type, handle, prio}; LaxityHint {type, handle, lax, lax_prio, crit_prio}  hint.h:47-77, :200-233
* status bookkeeping of LocalScheduler::UpdateStatus (sched/src/scheduler/local.cpp:237-407)
* decision rules of HPF (sched/src/policy/hpf.cpp:8-42) and LAX (sched/src/policy/lax.cpp:8-56)

Pinned against the compiled reference (oracle/_ref/sched_probe_ref) by tests/golden/make_sched_golden.py;
tests/test_sched_parity.py holds all three (this restatement, the reference's answers, the product) equal.
"""
from __future__ import annotations

import struct
import time

EV_HINT, EV_TERMINATE, EV_PROC_CREATE, EV_PROC_DESTROY, EV_XQ_CREATE, EV_XQ_DESTROY, EV_XQ_READY, EV_XQ_IDLE, EV_XQ_CONFIG = range(9)
EV_OP_COMPLETE = 11
HINT_PRIORITY, HINT_LAXITY = 1, 6
PRIORITY_MIN, PRIORITY_MAX, PRIORITY_DEFAULT = -255, 255, 0


def ev_proc_create(pid: int, cmdline: str = "") -> bytes:
    return struct.pack("<ii256s", EV_PROC_CREATE, pid, cmdline.encode()[:255])


def ev_proc_destroy(pid: int) -> bytes:
    return struct.pack("<ii", EV_PROC_DESTROY, pid)


def ev_xq_create(pid, handle, device, level=1, threshold=16, batch=8, update=False) -> bytes:
    return struct.pack("<iiQQi4xqq", EV_XQ_CONFIG if update else EV_XQ_CREATE, pid, handle, device, level, threshold, batch)


def ev_xq_destroy(pid, handle) -> bytes:
    return struct.pack("<iiQ", EV_XQ_DESTROY, pid, handle)


def ev_xq_ready(pid, handle, ready_time_us) -> bytes:
    return struct.pack("<iiQq", EV_XQ_READY, pid, handle, ready_time_us)


def ev_xq_idle(pid, handle) -> bytes:
    return struct.pack("<iiQ", EV_XQ_IDLE, pid, handle)


def _ev_hint(pid, hint: bytes) -> bytes:
    return struct.pack("<iiQ", EV_HINT, pid, 16 + len(hint)) + hint


def ev_hint_priority(pid, handle, prio) -> bytes:
    return _ev_hint(pid, struct.pack("<i4xQi4x", HINT_PRIORITY, handle, prio))


def ev_hint_laxity(pid, handle, lax_us, lax_prio, crit_prio) -> bytes:
    return _ev_hint(pid, struct.pack("<i4xQqii", HINT_LAXITY, handle, lax_us, lax_prio, crit_prio))


def now_us() -> int:
    return int(time.time() * 1e6)


class Model:
    """Status + policy, event by event; `decide()` returns {pid: (running, suspended)} like the newest
    Sched operation each process would have received."""

    def __init__(self, policy: str, scope: str = "GLOBAL"):
        self.policy, self.scope = policy, scope
        self.xq: dict[int, dict] = {}
        self.prio: dict[int, int] = {}
        self.lax: dict[int, tuple[int, int, int]] = {}
        self.last: dict[int, tuple[tuple, tuple]] = {}

    def _ensure(self, pid, handle):
        if handle not in self.xq:
            self.xq[handle] = dict(pid=pid, device=0, ready=False, suspended=False, ready_time=now_us())
        return self.xq[handle]

    def apply(self, ev: bytes) -> None:
        typ, pid = struct.unpack_from("<ii", ev)
        if typ == EV_HINT:
            htype = struct.unpack_from("<i", ev, 16)[0]
            if htype == HINT_PRIORITY and self.policy == "HPF":
                handle, prio = struct.unpack_from("<Qi", ev, 24)
                self.prio[handle] = max(PRIORITY_MIN, min(PRIORITY_MAX, prio))        # hpf.cpp:49-57
            elif htype == HINT_LAXITY and self.policy == "LAX":
                handle, lax, lp, cp = struct.unpack_from("<Qqii", ev, 24)
                self.lax[handle] = (-1 if lax < 0 else lax, lp, cp)                    # lax.cpp:64-71
        elif typ == EV_PROC_DESTROY:                                                   # local.cpp:263-275
            for h in [h for h, q in self.xq.items() if q["pid"] == pid]:
                del self.xq[h]
        elif typ in (EV_XQ_CREATE, EV_XQ_CONFIG):
            handle, device = struct.unpack_from("<QQ", ev, 8)
            self._ensure(pid, handle)["device"] = device
        elif typ == EV_XQ_DESTROY:
            self.xq.pop(struct.unpack_from("<Q", ev, 8)[0], None)
        elif typ == EV_XQ_READY:
            handle, t = struct.unpack_from("<Qq", ev, 8)
            q = self._ensure(pid, handle)
            q["ready"], q["ready_time"] = True, t
        elif typ == EV_XQ_IDLE:
            self._ensure(pid, struct.unpack_from("<Q", ev, 8)[0])["ready"] = False

    def decide(self, now: int | None = None) -> dict:
        now = now_us() if now is None else now
        susp = set()
        if self.policy == "HPF":
            top: dict[int, int] = {}
            for h, q in self.xq.items():
                if q["ready"]:
                    top[q["device"]] = max(top.get(q["device"], -10**9), self.prio.get(h, PRIORITY_DEFAULT))
            for h, q in self.xq.items():
                if self.prio.get(h, PRIORITY_DEFAULT) < top.get(q["device"], PRIORITY_MIN):
                    susp.add(h)
        else:
            key = (lambda q: q["device"]) if self.scope == "DEVICE" else (lambda q: 0)
            top = {}
            for h, q in self.xq.items():
                if not q["ready"]:
                    continue
                if h not in self.lax:
                    p = PRIORITY_DEFAULT
                else:
                    lax, lp, cp = self.lax[h]
                    p = lp if now < q["ready_time"] + lax else cp
                top[key(q)] = max(top.get(key(q), PRIORITY_MIN), p)
            for h, q in self.xq.items():
                p = PRIORITY_DEFAULT
                if h in self.lax:
                    lax, lp, cp = self.lax[h]
                    p = lp if (not q["ready"] or now < q["ready_time"] + lax) else cp
                if p < top.get(key(q), PRIORITY_MIN):
                    susp.add(h)
        for h, q in self.xq.items():
            q["suspended"] = h in susp
        per_pid: dict[int, tuple[list, list]] = {}
        for h, q in sorted(self.xq.items()):
            r, s = per_pid.setdefault(q["pid"], ([], []))
            (s if h in susp else r).append(h)
        for pid, (r, s) in per_pid.items():
            self.last[pid] = (tuple(r), tuple(s))
        return dict(self.last)
