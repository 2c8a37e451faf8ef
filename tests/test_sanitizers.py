"""The host runtime (XQueue, window worker, schedulers, IPC, host lane) under ThreadSanitizer and
AddressSanitizer + UBSan: the scenario runner is rebuilt from the sources with the sanitizer and a handful of
short scenarios — window, level-2 suspend/resume, drop, two queues under HPF and under the laxity policy,
locally and through a sanitized xserver — must finish without a single report."""
import os
import shutil
import signal
import subprocess
import time
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
CSRC = ROOT / "xsched_b200" / "csrc"
CXX = os.environ.get("XSCHED_CXX", "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++"))
SCENARIOS = [
    ["window", "4", "2", "40", "300"],
    ["suspend", "2", "60", "500"],
    ["drop", "2", "60", "500"],
    ["hpf", "2", "150", "500", "5", "1000", "12000", "16", "8", "LCL"],
    ["lax", "2", "150", "500", "4", "1000", "15000", "16", "8", "LCL", "3000"],
]


def build(tmp: Path, flag: str):
    """Objects are compiled once, in parallel, and linked into the scenario runner and the server."""
    from concurrent.futures import ThreadPoolExecutor
    units = {p: tmp / (p.parent.name + "_" + p.stem + ".o") for d in ("utils", "preempt", "sched", "hal_host") for p in sorted((CSRC / d).glob("*.cpp"))}
    units[ROOT / "oracle" / "lane_driver.cpp"] = tmp / "lane_driver.o"
    units[CSRC / "server" / "xserver.cpp"] = tmp / "xserver.o"
    units[CSRC / "server" / "http.cpp"] = tmp / "http.o"
    common = [CXX, "-std=c++20", "-O1", "-g", f"-fsanitize={flag}", "-pthread", f"-I{ROOT / 'include'}", f"-I{CSRC}"]

    def compile_one(item):
        src, obj = item
        return subprocess.run(common + ["-c", "-o", str(obj), str(src)], capture_output=True, text=True)
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        for r in pool.map(compile_one, units.items()):
            assert r.returncode == 0, r.stderr[-2000:]
    lane, srv = tmp / "lane_san", tmp / "xserver_san"
    core = [str(o) for s_, o in units.items() if s_.parent.name in ("utils", "preempt", "sched")]
    host = [str(o) for s_, o in units.items() if s_.parent.name == "hal_host"]
    for out, objs in ((lane, [str(tmp / "lane_driver.o")] + core + host), (srv, [str(tmp / "xserver.o"), str(tmp / "http.o")] + core)):
        r = subprocess.run(common + ["-o", str(out)] + objs + ["-ldl", "-lrt"], capture_output=True, text=True)
        if r.returncode != 0 and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
            pytest.skip(f"toolchain has no -fsanitize={flag} runtime")
        assert r.returncode == 0, r.stderr[-2000:]
    return lane, srv


def reports(text: str) -> int:
    return sum(text.count(k) for k in ("WARNING: ThreadSanitizer", "ERROR: AddressSanitizer", "runtime error:", "LeakSanitizer"))


@pytest.mark.parametrize("flag", ["thread", "address,undefined"])
def test_host_runtime_is_clean_under_the_sanitizer(tmp_path, flag):
    lane, srv = build(tmp_path, flag)
    env = dict(os.environ, XLOG_LEVEL="ERRO", TSAN_OPTIONS="halt_on_error=0", ASAN_OPTIONS="detect_leaks=1",
               XSCHED_IPC_NAMESPACE=f"san{os.getpid()}.")
    env.pop("XSCHED_SCHEDULER", None)
    for sc in SCENARIOS:
        r = subprocess.run([str(lane), *sc], capture_output=True, text=True, env=env, timeout=300)
        assert r.returncode == 0 and reports(r.stdout + r.stderr) == 0, (sc, (r.stdout + r.stderr)[-3000:])
    # two clients on two lanes through a sanitized server, blocking and polling receivers
    for spin in ("OFF", "ON"):
        e = dict(env, XSCHED_IPC_SPIN=spin)
        server = subprocess.Popen([str(srv), "LAX", "50000", "--status-interval-ms", "20"], stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True, env=e)
        try:
            assert "ready" in server.stdout.readline()
            clients = [subprocess.Popen([str(lane), "lax", "2", "150", "500", "4", "1000", "15000", "16", "8", "GLB", "3000"], stdout=subprocess.PIPE,
                                        stderr=subprocess.STDOUT, text=True, env=dict(e, LANE_ID=str(i))) for i in (0, 1)]
            outs = [c.communicate(timeout=300)[0] for c in clients]
            for c, o in zip(clients, outs):
                assert c.returncode == 0 and reports(o) == 0, o[-3000:]
            time.sleep(0.2)
        finally:
            server.send_signal(signal.SIGTERM)
            out = server.communicate(timeout=60)[0]
        assert reports(out) == 0, out[-3000:]
