"""The N > 1 shape of the path on CPU: several client processes (one per "device") under ONE xserver,
scheduled per device, plus bench.py's reference arm under a 2-rank torchrun (gloo control plane)."""
import json
import os
import signal
import subprocess
import sys
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
DRIVER = ROOT / "oracle" / "lane_driver_new"


@pytest.fixture()
def xserver():
    ns = f"t{os.getpid()}."
    env = dict(os.environ, XLOG_LEVEL="WARN", XSCHED_IPC_NAMESPACE=ns)
    env.pop("XSCHED_SCHEDULER", None)
    p = subprocess.Popen([str(LIB / "xserver"), "HPF", "50000", "--status-interval-ms", "50"], stdout=subprocess.PIPE, text=True, env=env)
    assert "ready" in p.stdout.readline()
    yield ns, p
    p.send_signal(signal.SIGTERM)
    p.wait(timeout=10)


def test_two_devices_one_server(xserver):
    ns, server = xserver
    for attempt in range(3):             # latency bounds assume an idle host: up to three attempts
        try:
            _two_devices_once(ns)
            break
        except AssertionError:
            if attempt == 2:
                raise
    # the server saw queues on two distinct devices
    time.sleep(0.2)
    server.send_signal(signal.SIGTERM)
    text = server.stdout.read()
    devices = set()
    for line in text.splitlines():
        if line.startswith("{"):
            for q in json.loads(line)["xqueues"]:
                devices.add(q["device"])
    assert len(devices) == 2, devices


def _two_devices_once(ns):
    env = dict(os.environ, XLOG_LEVEL="ERRO", XSCHED_IPC_NAMESPACE=ns)
    args = [str(DRIVER), "hpf", "2", "300", "1000", "8", "2000", "30000", "16", "8", "GLB"]
    procs = [subprocess.Popen(args, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=dict(env, LANE_ID=str(lane)))
             for lane in (0, 1)]
    outs = [p.communicate(timeout=120) for p in procs]
    for p, (out, err) in zip(procs, outs):
        assert p.returncode == 0, err[-1000:]
    res = [json.loads(out) for out, _ in outs]
    for r in res:
        # each device's high-priority command is served as if the other device did not exist
        # (median against the algorithmic bound; the tail only against a loose one: on a busy test host the lane
        # thread or a receiver can lose its core for a few milliseconds)
        assert r["hp"]["n"] == 8 and r["hp"]["p50_us"] <= 2000 + 1000 + 7000 and r["hp"]["p99_us"] <= 40000, r   # level 1 would sit near 14 ms
        assert r["flushed"] > 0


def test_client_death_is_detected(xserver):
    ns, server = xserver
    env = dict(os.environ, XLOG_LEVEL="ERRO", XSCHED_IPC_NAMESPACE=ns)
    # a client that is killed mid-run: the server must drop its queues (pidfd) and keep serving others
    victim = subprocess.Popen([str(DRIVER), "hpf", "2", "5000", "1000", "100", "2000", "30000", "16", "8", "GLB"],
                              stdout=subprocess.DEVNULL, stderr=subprocess.DEVNULL, env=env)
    time.sleep(0.5)
    victim.kill()
    victim.wait()
    time.sleep(0.3)
    r = subprocess.run([str(DRIVER), "hpf", "2", "200", "1000", "5", "2000", "30000", "16", "8", "GLB"], capture_output=True, text=True,
                       env=env, timeout=120)
    assert r.returncode == 0, r.stderr[-1000:]
    assert json.loads(r.stdout)["hp"]["n"] == 5
    server.send_signal(signal.SIGTERM)
    lines = [json.loads(l) for l in server.stdout.read().splitlines() if l.startswith("{")]
    assert lines and lines[-1]["xqueues"] == []            # nothing left behind by the dead client


@pytest.mark.skipif(not (ROOT / "oracle" / "_ref" / "lane_driver_ref").exists(), reason="compiled reference core not present")
def test_bench_reference_arm_two_ranks_gloo():
    port = 29500 + os.getpid() % 1000
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                        "--master-port", str(port), str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "20", "--warmup", "3"],
                       capture_output=True, text=True, timeout=300, cwd=ROOT)
    assert r.returncode == 0, r.stderr[-2000:]
    lines = [json.loads(l) for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1                                   # rank 0 alone prints
    line = lines[0]
    assert line["impl"] == "reference" and line["n_gpus"] == 2 and line["metric"] == "hp_p99_latency_vs_standalone"
    assert line["cpu_baseline"]["kind"] == "reference" and line["value"] > 1.0
