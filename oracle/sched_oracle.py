"""Pure-Python restatement of the scheduling half of the path (TEST INFRASTRUCTURE).

* record layouts of the agent -> server events and hints, as the reference defines them:
    EventMeta {int32 type; int32 pid}                      sched/include/xsched/sched/protocol/event.h:33-37
    XQueueCreate/ConfigUpdate {meta, handle, device, level, threshold, batch}   event.h:146-205, :290-349
    XQueueDestroy/Idle {meta, handle}; XQueueReady {meta, handle, ready_time_us}  event.h:207-288
    ProcessCreate {meta, char cmdline[256]}; ProcessDestroy {meta}               event.h:101-143
    HintEvent {meta, size_t size, hint bytes}                                    event.h:55-84
    PriorityHint {type, handle, prio}; LaxityHint {type, handle, lax, lax_prio, crit_prio}  hint.h:47-77, :200-233
* status bookkeeping of LocalScheduler::UpdateStatus (sched/src/scheduler/local.cpp:237-407)
* decision rules of HPF (sched/src/policy/hpf.cpp:8-42) and LAX (sched/src/policy/lax.cpp:8-56), and of the
  other policies: HHPF hhpf.cpp:8-30, CHPF chpf.cpp:10-66, UP up.cpp:6-164, PUP pup.cpp:7-200,
  KEDF kedf.cpp:11-47, AWF awf.cpp:6-51, CFS cfs.cpp:10-124, MLFQ mlfq.cpp:7-173

Pinned against the compiled reference (oracle/_ref/sched_probe_ref) by tests/golden/make_sched_golden.py;
tests/test_sched_parity.py holds all three (this restatement, the reference's answers, the product) equal.
"""
from __future__ import annotations

import struct
import time

EV_HINT, EV_TERMINATE, EV_PROC_CREATE, EV_PROC_DESTROY, EV_XQ_CREATE, EV_XQ_DESTROY, EV_XQ_READY, EV_XQ_IDLE, EV_XQ_CONFIG = range(9)
EV_OP_COMPLETE = 11
HINT_PRIORITY, HINT_UTILIZATION, HINT_TIMESLICE, HINT_DEADLINE, HINT_KDEADLINE, HINT_LAXITY, HINT_WINDOW_ACTIVE = 1, 2, 3, 4, 5, 6, 7
UTILIZATION_MIN, UTILIZATION_MAX, UTILIZATION_DEFAULT = 0, 100, 100
TIMESLICE_MIN, TIMESLICE_MAX, TIMESLICE_DEFAULT = 100, 10_000_000, 5000
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


def ev_hint_utilization(pid, target_pid, handle, util) -> bytes:
    return _ev_hint(pid, struct.pack("<iiQi4x", HINT_UTILIZATION, target_pid, handle, util))


def ev_hint_timeslice(pid, ts_us) -> bytes:
    return _ev_hint(pid, struct.pack("<i4xq", HINT_TIMESLICE, ts_us))


def ev_hint_deadline(pid, handle, ddl_us) -> bytes:
    return _ev_hint(pid, struct.pack("<i4xQq", HINT_DEADLINE, handle, ddl_us))


def ev_hint_kdeadline(pid, k) -> bytes:
    return _ev_hint(pid, struct.pack("<i4xQ", HINT_KDEADLINE, k))


def ev_hint_window_active(pid, active_pid, display) -> bytes:
    return _ev_hint(pid, struct.pack("<iiQ", HINT_WINDOW_ACTIVE, active_pid, display))


def linux_priority(pid: int) -> int:
    """chpf.cpp:16-33: third field of the first line of /proc/<pid>/sched that contains "prio"."""
    try:
        with open(f"/proc/{pid}/sched") as f:
            for line in f:
                if "prio" in line:
                    tok = line.split()
                    v = int(tok[2]) if len(tok) > 2 and tok[2].lstrip("-").isdigit() else 0
                    return -v if v >= 100 else v
    except OSError:
        pass
    return 0


def now_us() -> int:
    return int(time.time() * 1e6)


class Model:
    """Status + policy, event by event; `decide()` returns {pid: (running, suspended)} like the newest
    Sched operation each process would have received.  A policy yields ordered verdicts (handle, suspend);
    a queue that gets none stays as it is."""

    def __init__(self, policy: str, scope: str = "GLOBAL"):
        self.policy, self.scope = policy, scope
        self.xq: dict[int, dict] = {}
        self.procs: set[int] = set()
        self.prio: dict[int, int] = {}
        self.lax: dict[int, tuple[int, int, int]] = {}
        self.last: dict[int, tuple[tuple, tuple]] = {}
        # UP / PUP / KEDF / AWF / CFS / MLFQ state
        self.utils: dict[int, int] = {}            # by handle (UP) or pid (PUP)
        self.timeslice = TIMESLICE_DEFAULT
        self.current, self.current_end = 0, 0
        self.runq: list[dict] = []
        self.slice_end = -(1 << 62)
        self.deadlines: dict[int, int] = {}
        self.k = 1
        self.active: set[int] = set()
        self.by_display: dict[int, int] = {}
        self.nodes: dict[int, dict] = {}
        self.timers: list[int] = []                # absolute times at which the policy wants another round

    def _ensure(self, pid, handle):
        if handle not in self.xq:
            self.xq[handle] = dict(pid=pid, device=0, ready=False, suspended=False, ready_time=now_us())
        return self.xq[handle]

    def apply(self, ev: bytes) -> None:
        typ, pid = struct.unpack_from("<ii", ev)
        if typ == EV_HINT:
            self._hint(ev)
        elif typ == EV_PROC_CREATE:
            self.procs.add(pid)
        elif typ == EV_PROC_DESTROY:                                                   # local.cpp:263-275
            self.procs.discard(pid)
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

    def _hint(self, ev: bytes) -> None:
        htype = struct.unpack_from("<i", ev, 16)[0]
        P = self.policy
        if htype == HINT_PRIORITY and P in ("HPF", "HHPF"):
            handle, prio = struct.unpack_from("<Qi", ev, 24)
            self.prio[handle] = max(PRIORITY_MIN, min(PRIORITY_MAX, prio))            # hpf.cpp:49-57
        elif htype == HINT_PRIORITY and P == "CFS":
            handle, prio = struct.unpack_from("<Qi", ev, 24)
            self._cfs_node(handle)["weight"] = 1024.0 * 1.2 ** prio                   # cfs.cpp:117-120
        elif htype == HINT_LAXITY and P == "LAX":
            handle, lax, lp, cp = struct.unpack_from("<Qqii", ev, 24)
            self.lax[handle] = (-1 if lax < 0 else lax, lp, cp)                        # lax.cpp:64-71
        elif htype == HINT_UTILIZATION and P in ("UP", "PUP"):
            target, handle, util = struct.unpack_from("<iQi", ev, 20)
            if UTILIZATION_MIN <= util <= UTILIZATION_MAX:
                if P == "UP":
                    self.utils[handle] = util                                          # up.cpp:100-110
                elif target != 0:
                    self.utils[target] = util                                          # pup.cpp:102-114
        elif htype == HINT_TIMESLICE and P in ("UP", "PUP"):
            ts = struct.unpack_from("<q", ev, 24)[0]
            if P == "UP" or TIMESLICE_MIN <= ts <= TIMESLICE_MAX:                      # only PUP checks the range
                self.timeslice = ts
        elif htype == HINT_DEADLINE and P == "KEDF":
            handle, ddl = struct.unpack_from("<Qq", ev, 24)
            self.deadlines[handle] = ddl
        elif htype == HINT_KDEADLINE and P == "KEDF":
            k = struct.unpack_from("<Q", ev, 24)[0]
            if k >= 1:
                self.k = k
        elif htype == HINT_WINDOW_ACTIVE and P == "AWF":
            apid, display = struct.unpack_from("<iQ", ev, 20)
            if apid != 0:
                if display in self.by_display:
                    self.active.discard(self.by_display[display])
                self.active.add(apid)
                self.by_display[display] = apid

    # -- helpers --------------------------------------------------------------------------------
    def _items(self):
        return sorted(self.xq.items())

    def _proc_sets(self, pid):
        run = [h for h, q in self._items() if q["pid"] == pid and not q["suspended"]]
        sus = [h for h, q in self._items() if q["pid"] == pid and q["suspended"]]
        return run, sus

    def _all_pids(self):
        return sorted(self.procs | {q["pid"] for q in self.xq.values()})

    # -- policies -------------------------------------------------------------------------------
    def _hpf(self, now, per_device=True, prio_of=None):
        prio_of = prio_of or (lambda h, q: self.prio.get(h, PRIORITY_DEFAULT))
        key = (lambda q: q["device"]) if per_device else (lambda q: 0)
        top: dict[int, int] = {}
        for h, q in self._items():
            if q["ready"]:
                top[key(q)] = max(top.get(key(q), -10**9), prio_of(h, q))
        return [(h, prio_of(h, q) < top.get(key(q), PRIORITY_MIN)) for h, q in self._items()]

    def _chpf(self, now):
        pp = {pid: linux_priority(pid) for pid in self._all_pids()}
        return self._hpf(now, True, lambda h, q: pp.get(q["pid"], 0))

    def _lax(self, now):
        key = (lambda q: q["device"]) if self.scope == "DEVICE" else (lambda q: 0)
        top = {}
        for h, q in self._items():
            if not q["ready"]:
                continue
            if h not in self.lax:
                p = PRIORITY_DEFAULT
            else:
                lax, lp, cp = self.lax[h]
                p = lp if now < q["ready_time"] + lax else cp
                if now < q["ready_time"] + lax:
                    self.timers.append(q["ready_time"] + lax)                          # lax.cpp:37-47
            top[key(q)] = max(top.get(key(q), PRIORITY_MIN), p)
        out = []
        for h, q in self._items():
            p = PRIORITY_DEFAULT
            if h in self.lax:
                lax, lp, cp = self.lax[h]
                p = lp if (not q["ready"] or now < q["ready_time"] + lax) else cp
            out.append((h, p < top.get(key(q), PRIORITY_MIN)))
        return out

    def _up_budget(self, util):
        total = sum(self.utils.values())
        return TIMESLICE_DEFAULT if total == 0 else self.timeslice * util // total

    def _up(self, now):
        for h in [h for h in self.utils if h not in self.xq]:
            del self.utils[h]
        if self.current and self.current not in self.xq:
            self.current = 0
        if not self.utils:
            return []
        out = []

        def hand_any():
            self.current = 0
            for h, q in self._items():
                if self.current or not q["ready"] or h not in self.utils:
                    out.append((h, True))
                    continue
                out.append((h, False))
                self.current, self.current_end = h, now + self._up_budget(self.utils[h])
                self.timers.append(self.current_end)

        def hand_to(h):
            out.extend((o, True) for o, _ in self._items() if o != h)
            out.append((h, False))
            self.current, self.current_end = h, now + self._up_budget(self.utils[h])
            self.timers.append(self.current_end)

        if not self.current:
            hand_any()
            return out
        if now < self.current_end and self.xq[self.current]["ready"]:
            return out
        order = sorted(self.utils)
        i = order.index(self.current)
        for h in order[i + 1:] + order[:i]:
            if self.xq[h]["ready"]:
                hand_to(h)
                return out
        self.current = 0
        return out

    def _pup(self, now):
        pids = self._all_pids()
        for p in [p for p in self.utils if p not in pids]:
            del self.utils[p]
        owns = lambda pid: any(q["pid"] == pid for q in self.xq.values())
        ready = lambda pid: any(q["pid"] == pid and q["ready"] for q in self.xq.values())
        self.runq = [e for e in self.runq if e["pid"] in pids and owns(e["pid"])]
        for e in self.runq:
            e["ready"] = ready(e["pid"])
        queued = {e["pid"] for e in self.runq}
        for pid in pids:
            if owns(pid) and pid not in queued:
                self.runq.append(dict(pid=pid, ready=ready(pid), running=False, budget=0))
        if not self.runq or not any(e["ready"] for e in self.runq):
            return []

        def fresh(pid):
            total = sum(self.utils.get(e["pid"], UTILIZATION_DEFAULT) for e in self.runq)
            return 0 if total == 0 else self.timeslice * len(self.runq) * self.utils.get(pid, UTILIZATION_DEFAULT) // total

        def turn_budget(e):
            f, b = fresh(e["pid"]), e["budget"]
            if b > f:
                b = int(f + (b - f) * 0.9)
            return b + f

        def rotate(budget):
            e = self.runq.pop(0)
            e["running"], e["budget"] = False, budget
            self.runq.append(e)

        if self.runq[0]["running"]:
            left = self.slice_end > now
            if left and self.runq[0]["ready"]:
                return []
            rotate(self.slice_end - now if left else 0)
        while not self.runq[0]["ready"]:
            rotate(turn_budget(self.runq[0]))
        head = self.runq[0]
        self.slice_end = now + turn_budget(head)
        self.timers.append(self.slice_end)
        out = []
        for e in self.runq:
            run, sus = self._proc_sets(e["pid"])
            if e["pid"] == head["pid"]:
                out.extend((h, False) for h in sus)
            else:
                out.extend((h, True) for h in run)
            e["running"] = e["pid"] == head["pid"]
        return out

    def _kedf(self, now):
        never = 1 << 62
        order = sorted(((q["ready_time"] + self.deadlines[h]) if (q["ready"] and h in self.deadlines) else never, h) for h, q in self._items())
        return [(h, i >= self.k) for i, (_, h) in enumerate(order)]

    def _awf(self, now):
        wants = any(q["ready"] and q["pid"] in self.active for q in self.xq.values())
        return [(h, wants and q["pid"] not in self.active) for h, q in self._items()]

    def _cfs_node(self, h):
        return self.nodes.setdefault(h, dict(weight=1024.0, vruntime=0.0, last=0, running=False))

    def _cfs(self, now):
        for h, q in self._items():
            n = self.nodes.get(h)
            if n and n["running"]:
                n["vruntime"] += (now - n["last"]) * (1024.0 / n["weight"])
        floor: dict[int, float] = {}
        for h, q in self._items():
            if q["ready"] and h in self.nodes:
                floor[q["device"]] = min(floor.get(q["device"], float("inf")), self.nodes[h]["vruntime"])
        pick: dict[int, int] = {}
        for h, q in self._items():
            if not q["ready"]:
                continue
            if h not in self.nodes:
                n = self._cfs_node(h)
                n["last"] = now
                n["vruntime"] = floor.get(q["device"], 0.0)
                floor.setdefault(q["device"], n["vruntime"])
            d = q["device"]
            if d not in pick or self.nodes[h]["vruntime"] < self.nodes[pick[d]]["vruntime"]:
                pick[d] = h
        out = []
        for h, q in self._items():
            n = self._cfs_node(h)
            if not q["ready"]:
                n["running"] = False
                continue
            if pick[q["device"]] == h:
                if not n["running"]:
                    out.append((h, False))
                n["running"], n["last"] = True, now
            else:
                out.append((h, True))
                n["running"] = False
        if any(q["ready"] for q in self.xq.values()):
            self.timers.append(now + 1000)
        return out

    def _mlfq(self, now):
        for h, q in self._items():
            if h not in self.nodes:
                self.nodes[h] = dict(level=0, running=False, was_ready=False, since=now, pending=0, pending_from=now, used=0, resumed=now)
            n = self.nodes[h]
            if q["ready"] and not n["was_ready"]:
                n["pending_from"] = now
            n["was_ready"] = q["ready"]
        count: dict[tuple, int] = {}
        for h, q in self._items():
            if q["ready"]:
                k = (q["device"], self.nodes[h]["level"])
                count[k] = count.get(k, 0) + 1
        out = []
        for h, q in self._items():
            if not q["ready"]:
                continue
            n = self.nodes[h]
            if not n["running"]:
                n["pending"] += now - n["pending_from"]
                n["pending_from"] = now
            else:
                n["used"] += now - n["resumed"]
                n["resumed"] = now
            peers = count.get((q["device"], n["level"]), 0)
            discount = 0.9 / peers if peers > 1 else 1.0
            if (now - n["since"]) - n["pending"] * discount > 100000:
                n["level"] = max(0, n["level"] - 1)
                n["since"], n["pending"], n["used"] = now, 0, 0
            if n["running"] and n["used"] >= (10000 << n["level"]):
                n["level"] = min(3, n["level"] + 1)
                n["since"], n["used"], n["pending"] = now, 0, 0
                n["running"] = False
                out.append((h, True))
                n["pending_from"] = now
        pick: dict[int, int] = {}
        for h, q in self._items():
            if not q["ready"]:
                continue
            n, d = self.nodes[h], q["device"]
            if d not in pick:
                pick[d] = h
                continue
            b = self.nodes[pick[d]]
            if n["level"] < b["level"] or (n["level"] == b["level"] and n["pending"] > b["pending"]):
                pick[d] = h
        for h, q in self._items():
            n = self.nodes[h]
            if not q["ready"]:
                n["running"] = False
                continue
            if pick[q["device"]] == h:
                if not n["running"]:
                    out.append((h, False))
                    n["running"], n["pending_from"] = True, now
                n["resumed"] = now
            elif n["running"]:
                out.append((h, True))
                n["running"], n["pending_from"] = False, now
        if any(q["ready"] for q in self.xq.values()):
            self.timers.append(now + 5000)
        return out

    def advance(self, now: int, until: int) -> int:
        """Let virtual time pass from `now` to `until`, running one round at every timer that falls due."""
        while True:
            due = [t for t in self.timers if t <= until]
            if not due:
                return until
            t = max(now, min(due))
            self.timers = [x for x in self.timers if x > t]
            self.decide(t)
            now = t

    def snapshot(self) -> dict:
        """{pid: (running, suspended)} as of the last round."""
        per_pid: dict[int, tuple[list, list]] = {}
        for h, q in self._items():
            r, s = per_pid.setdefault(q["pid"], ([], []))
            (s if q["suspended"] else r).append(h)
        for pid, (r, s) in per_pid.items():
            self.last[pid] = (tuple(r), tuple(s))
        return dict(self.last)

    def decide(self, now: int | None = None) -> dict:
        now = now_us() if now is None else now
        rule = {"HPF": self._hpf, "HHPF": lambda t: self._hpf(t, per_device=False), "CHPF": self._chpf, "LAX": self._lax, "UP": self._up,
                "PUP": self._pup, "KEDF": self._kedf, "AWF": self._awf, "CFS": self._cfs, "MLFQ": self._mlfq}[self.policy]
        for h, suspend in rule(now):
            if h in self.xq:
                self.xq[h]["suspended"] = suspend
        return self.snapshot()
