"""The scheduling server's control interface (HTTP/JSON) and `xcli`, on CPU: a client process with two XQueues on the
host-only lane runs under an xserver; the routes must list its queues with the reference's field names, change
a queue's launch configuration through a Config operation, accept hints that change the policy's decisions, swap
the policy, and answer malformed requests with the reference's status codes (service/server/src/server.cpp:228-544)."""
import json
import os
import signal
import socket
import subprocess
import time
import urllib.error
import urllib.request
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
DRIVER = ROOT / "oracle" / "lane_driver_new"
XCLI = LIB / "xcli"


def free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def call(port, method, target, body=None):
    req = urllib.request.Request(f"http://127.0.0.1:{port}{target}", data=body.encode() if body is not None else (b"" if method == "POST" else None), method=method)
    try:
        with urllib.request.urlopen(req, timeout=5) as r:
            text = r.read().decode()
            return r.status, json.loads(text) if text else None
    except urllib.error.HTTPError as e:
        text = e.read().decode()
        return e.code, json.loads(text) if text else None


@pytest.fixture()
def served():
    ns = f"ctl{os.getpid()}."
    port = free_port()
    env = dict(os.environ, XLOG_LEVEL="WARN", XSCHED_IPC_NAMESPACE=ns)
    env.pop("XSCHED_SCHEDULER", None)
    server = subprocess.Popen([str(LIB / "xserver"), "HPF", str(port)], stdout=subprocess.PIPE, text=True, env=env)
    ready = server.stdout.readline()
    assert "ready" in ready and f"http={port}" in ready, ready
    # a client with a low- and a high-priority XQueue on one host lane, busy for several seconds
    client = subprocess.Popen([str(DRIVER), "hpf", "1", "6000", "1000", "400", "2000", "15000", "16", "8", "GLB"], stdout=subprocess.PIPE,
                              stderr=subprocess.PIPE, text=True, env=dict(env, XLOG_LEVEL="ERRO"))
    deadline = time.time() + 10
    while time.time() < deadline:
        st, body = call(port, "GET", "/xqueues")
        if st == 200 and len(body["xqueues"]) >= 2:
            break
        time.sleep(0.05)
    yield port, client
    client.kill()
    client.wait()
    server.send_signal(signal.SIGTERM)
    server.wait(timeout=10)


def test_list_get_config_hint_and_policy_routes(served):
    port, client = served
    st, body = call(port, "GET", "/xqueues")
    assert st == 200 and len(body["xqueues"]) == 2
    q = body["xqueues"][0]
    assert set(q) == {"handle", "device", "level", "pid", "threshold", "batch_size", "ready", "suspended"}       # the reference's JSON schema
    assert q["pid"] == client.pid and q["threshold"] == 16 and q["batch_size"] == 8 and q["level"] == 1
    assert body["processes"] == [{"pid": client.pid, "cmdline": body["processes"][0]["cmdline"]}] and "lane_driver" in body["processes"][0]["cmdline"]

    st, one = call(port, "GET", f"/xqueue/{q['handle']:x}")
    assert st == 200 and one["xqueue"]["handle"] == q["handle"] and one["process"]["pid"] == client.pid
    assert call(port, "GET", "/xqueue/123456")[0] == 404
    assert call(port, "GET", "/xqueue/zz")[0] == 400
    assert call(port, "GET", "/nothing")[0] == 404

    # configuration change: reaches the client as a Config operation, comes back in the next listing.  As in the
    # reference the XQueue drains before its window changes (preempt/src/xqueue/async_xqueue.cpp:201-204), so the
    # queue that takes it here is the high-priority one, which is idle between its requests.
    idle_seen = {}
    deadline = time.time() + 3
    while time.time() < deadline and not idle_seen:
        for x in call(port, "GET", "/xqueues")[1]["xqueues"]:
            if not x["ready"]:
                idle_seen[x["handle"]] = x
        time.sleep(0.005)
    assert idle_seen, "no queue was ever idle"
    q = next(iter(idle_seen.values()))
    assert call(port, "POST", f"/config/{q['handle']:x}?threshold=4&batch_size=2") == (200, {"info": "success"})
    deadline = time.time() + 5
    while time.time() < deadline:
        now = call(port, "GET", f"/xqueue/{q['handle']:x}")[1]["xqueue"]
        if now["threshold"] == 4:
            break
        time.sleep(0.05)
    assert now["threshold"] == 4 and now["batch_size"] == 2
    assert call(port, "POST", f"/config/{q['handle']:x}") == (200, {"warning": "no change"})
    assert call(port, "POST", f"/config/{q['handle']:x}?level=9") == (400, {"error": "invalid level"})
    assert call(port, "POST", f"/config/{q['handle']:x}?threshold=0") == (400, {"error": "invalid command threshold"})
    assert call(port, "POST", f"/config/{q['handle']:x}?threshold=2&batch_size=5")[0] == 400
    assert call(port, "POST", "/config/abcdef?threshold=4") == (404, {"error": "XQueue not found"})

    # policy: query, swap, swap back; an out-of-range number is refused
    st, pol = call(port, "GET", "/policy")
    assert st == 200 and pol["name"] == "HPF"
    hpf = pol["policy"]
    assert call(port, "POST", "/policy?policy=999")[0] == 400 and call(port, "POST", "/policy")[0] == 400
    others = [p for p in range(1, 16) if p != hpf and call(port, "POST", f"/policy?policy={p}")[0] == 200]
    assert others, "no other policy accepted"
    assert call(port, "GET", "/policy")[1]["policy"] == others[-1]
    assert call(port, "POST", f"/policy?policy={hpf}") == (200, {"info": "success"})

    # hints: validation as in the reference, and a priority hint that changes who is suspended
    assert call(port, "POST", "/hint", "not json")[0] == 400
    assert call(port, "POST", "/hint", "{}") == (400, {"error": "missing hint type"})
    assert call(port, "POST", "/hint", '{"hint_type": 99}') == (400, {"error": "invalid hint type"})
    assert call(port, "POST", "/hint", '{"hint_type": 1, "priority": 3}') == (400, {"error": "invalid handle"})
    assert call(port, "POST", "/hint", json.dumps({"hint_type": 1, "handle": q["handle"]})) == (400, {"error": "missing priority"})
    assert call(port, "POST", "/hint", json.dumps({"hint_type": 1, "handle": q["handle"], "priority": 1000})) == (400, {"error": "invalid priority"})
    assert call(port, "POST", "/hint", '{"hint_type": 3, "timeslice": 5000}') == (200, {"info": "success"})
    assert call(port, "POST", "/hint", json.dumps({"hint_type": 2, "pid": client.pid, "utilization": 50})) == (200, {"info": "success"})
    qs = call(port, "GET", "/xqueues")[1]["xqueues"]
    for x in qs:       # raise both queues far above anything the client hinted, the first one highest
        assert call(port, "POST", "/hint", json.dumps({"hint_type": 1, "handle": x["handle"], "priority": 200 if x is qs[0] else 100})) == (200, {"info": "success"})
    # while both are ready, the second one must now be the suspended one at some point
    seen = False
    deadline = time.time() + 5
    while time.time() < deadline and not seen:
        cur = {x["handle"]: x for x in call(port, "GET", "/xqueues")[1]["xqueues"]}
        a, b = cur.get(qs[0]["handle"]), cur.get(qs[1]["handle"])
        seen = bool(a and b and a["ready"] and not a["suspended"] and b["suspended"])
        time.sleep(0.01)
    assert seen, "the priority hint given over the control interface never showed in the schedule"


def test_xcli_commands(served):
    port, client = served
    base = [str(XCLI), "-p", str(port)]
    r = subprocess.run(base + ["list"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0, r.stderr
    lines = r.stdout.strip().splitlines()
    assert lines[0].split()[:6] == ["PID", "DEV", "XQUEUE", "STAT", "SCHED", "LV"] and lines[-1] == "2 XQueue(s)"
    assert all(l.split()[0] == str(client.pid) for l in lines[1:3])
    handle = lines[1].split()[2]
    r = subprocess.run(base + ["config", "-x", handle, "-t", "6", "-b", "3"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0 and json.loads(r.stdout) == {"info": "success"}
    r = subprocess.run(base + ["policy", "-q"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0 and json.loads(r.stdout)["name"] == "HPF"
    r = subprocess.run(base + ["policy", "-s", "-n", "LAX"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0 and json.loads(r.stdout) == {"info": "success"}
    assert json.loads(subprocess.run(base + ["policy", "-q"], capture_output=True, text=True, timeout=20).stdout)["name"] == "LAX"
    r = subprocess.run(base + ["policy", "-s", "-n", "NOPE"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 1
    r = subprocess.run(base + ["hint", "-x", handle, "-p", "7"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0 and json.loads(r.stdout) == {"info": "success"}
    r = subprocess.run(base + ["hint", "-t", "2000"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 0
    r = subprocess.run([str(XCLI), "-p", str(free_port()), "list"], capture_output=True, text=True, timeout=20)
    assert r.returncode == 1 and "cannot reach" in r.stderr
