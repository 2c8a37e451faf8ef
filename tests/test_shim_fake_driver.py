"""The libcuda interposer and the CUDA HAL on a machine WITHOUT a GPU: a host-only stand-in for the driver
(tests/fake_cuda/fake_cuda.cpp: streams are threads, kernels are host functions) sits where the real
libcuda.so.1 would, and a driver-API program (tests/fake_cuda/driver_app.cpp) runs on it directly and under
the interposer.  The program checks every result itself and prints a checksum; under the interposer the
checksum must be the same and every stream operation must have gone through an XQueue.  The same stack is
also rebuilt under ThreadSanitizer and must run without a report."""
import json
import os
import shutil
import subprocess
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
LIB = ROOT / "xsched_b200" / "lib"
FAKE_DIR = ROOT / "tests" / "fake_cuda"
FAKE, APP = FAKE_DIR / "libcuda_fake.so", FAKE_DIR / "driver_app"
CSRC = ROOT / "xsched_b200" / "csrc"
CUDA_INC = Path(os.environ.get("CUDA_HOME", "/usr/local/cuda")) / "include"
CXX = os.environ.get("XSCHED_CXX", "/usr/bin/g++" if Path("/usr/bin/g++").exists() else (shutil.which("g++") or "g++"))


@pytest.fixture(scope="module", autouse=True)
def built():
    if not (FAKE.exists() and APP.exists()):
        from xsched_b200 import build
        build.build_host()
        build.build_fake_driver()
    assert FAKE.exists() and APP.exists()


def as_libcuda(tmp: Path, target: Path) -> Path:
    d = tmp / target.stem
    d.mkdir(exist_ok=True)
    for name in ("libcuda.so.1", "libcuda.so"):
        if not (d / name).exists():
            os.symlink(target, d / name)
    return d


def run_app(libdir: Path, fake: Path, app: Path, rounds: int = 30, **extra):
    """Run `app` with `libdir` (holding libcuda.so.1) first on the loader path."""
    env = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
    env.update(FAKE_CUDA_LIB=str(fake), LD_LIBRARY_PATH=f"{libdir}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""), XLOG_LEVEL="WARN")
    env.update({k: str(v) for k, v in extra.items()})
    return subprocess.run([str(app), str(rounds)], capture_output=True, text=True, env=env, timeout=300)


@pytest.mark.parametrize("level,threshold,batch", [(1, 4, 2), (1, 1, 1), (2, 16, 8)])
def test_driver_program_under_the_interposer_without_a_gpu(tmp_path, level, threshold, batch):
    plain = run_app(as_libcuda(tmp_path, FAKE), FAKE, APP)
    assert plain.returncode == 0 and plain.stdout.startswith("OK "), plain.stdout + plain.stderr
    stats = tmp_path / "stats.json"
    r = run_app(as_libcuda(tmp_path, LIB / "libshimcuda.so"), FAKE, APP, XSCHED_CUDA_LIB=FAKE, XSCHED_AUTO_XQUEUE="ON", XSCHED_POLICY="HPF",
                XSCHED_AUTO_XQUEUE_LEVEL=level, XSCHED_AUTO_XQUEUE_THRESHOLD=threshold, XSCHED_AUTO_XQUEUE_BATCH_SIZE=batch,
                XSCHED_SHIM_STATS_FILE=stats)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["streams_with_xqueue"] == 4            # two worker streams, the blocking stream, the short-lived one
    # 3 launches per round + 5 on the blocking stream + 5 between the graph launches go through XQueues; the 5 on
    # the legacy stream go straight to the driver after the blocking streams' XQueues were drained, and so do the
    # 3 launches recorded while a stream was capturing (a failed cuStreamEndCapture in between must not end the bypass)
    assert st["launches_queued"] == 30 * 3 + 5 + 5 and st["launches_direct"] == 5 + 3 and st["launches_blocking"] == 0
    assert st["graphs_queued"] == 5 and st["calls_queued"] == 5
    assert st["copies_queued"] == 30 * 6 + 3 and st["copies_direct"] == 5
    assert st["copies_waited"] == 30 * 2 + 3         # every copy into pageable memory on an XQueue stream
    assert st["events_queued"] == 30 + 1


def test_xsched_aware_program_on_the_cuda_hal_without_a_gpu(tmp_path):
    """XQueue C API + CudaQueueCreate on fake streams, in-process HPF, level 1 with window (4, 2): every command
    runs exactly once, a suspension waits at most for the window (4 x 500 us) and nothing of the suspended queue
    runs until it is resumed (the program checks that itself)."""
    hal_app = FAKE_DIR / "hal_app"
    assert hal_app.exists(), "tests/fake_cuda/hal_app not built (python -m xsched_b200.build)"
    r = run_app(as_libcuda(tmp_path, FAKE), FAKE, hal_app, XSCHED_CUDA_LIB=FAKE)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["ran"] == res["expected"]
    assert res["suspend_max_us"] <= 4 * 500 + 15000
    assert 300 <= res["hp_min_us"] <= 300 + 4000 and res["hp_max_us"] <= 60000       # (the maximum only loosely: a busy host)


def test_level2_preempt_and_resume_on_the_cuda_hal_without_a_gpu(tmp_path):
    """Level 2 of the CUDA HAL with fake preemptible tasks (tests/fake_cuda/fake_xpk.cpp stands in for libxpk): the
    low-priority queue is deactivated for every high-priority request, tasks stop at a tile boundary and are
    relaunched from their cursor; every tile of every task must have run exactly once."""
    app = FAKE_DIR / "level2_app"
    assert app.exists(), "tests/fake_cuda/level2_app not built (python -m xsched_b200.build)"
    r = run_app(as_libcuda(tmp_path, FAKE), FAKE, app, XSCHED_CUDA_LIB=FAKE)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    res = json.loads(r.stdout.strip().splitlines()[-1])
    assert res["finished"] == res["expected"] and res["bad_tiles"] == 0, res
    assert res["preemptions"] > 10 and res["relaunches"] >= res["preemptions"] and res["deactivations"] >= 10, res
    assert res["hp_p50_us"] < 300 + 200 + 5000            # about one tile, never one 8 ms task


def test_level2_low_priority_process_preempted_by_a_transparent_process(tmp_path):
    """The deployment shape of the benchmark's inference configuration, without a GPU: a low-priority process that
    uses the XQueue API with preemptible (fake) tasks at level 2, a high-priority XSched-unaware process under the
    interposer, one xserver with HPF.  Every request of the latter deactivates the former's queue; its tasks are
    relaunched from their cursors and every tile still runs exactly once."""
    import signal
    import time
    ns = f"l2{os.getpid()}."
    srv_env = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
    srv_env.update(XSCHED_IPC_NAMESPACE=ns, XLOG_LEVEL="WARN")
    server = subprocess.Popen([str(LIB / "xserver"), "HPF", "50000"], stdout=subprocess.PIPE, text=True, env=srv_env)
    lp = None
    try:
        assert "ready" in server.stdout.readline()
        common = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
        common.update(FAKE_CUDA_LIB=str(FAKE), XSCHED_CUDA_LIB=str(FAKE), XLOG_LEVEL="WARN", XSCHED_IPC_NAMESPACE=ns, XSCHED_SCHEDULER="GLB")
        lp_env = dict(common, LD_LIBRARY_PATH=f"{as_libcuda(tmp_path, FAKE)}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""), L2_LP_ONLY="1", L2_ITERATIONS="90")
        lp = subprocess.Popen([str(FAKE_DIR / "level2_app")], stdout=subprocess.PIPE, text=True, env=lp_env)
        assert lp.stdout.readline().startswith("READY")
        hp_env = dict(common, LD_LIBRARY_PATH=f"{as_libcuda(tmp_path, LIB / 'libshimcuda.so')}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""),
                      XSCHED_AUTO_XQUEUE="ON", XSCHED_AUTO_XQUEUE_LEVEL="1", XSCHED_AUTO_XQUEUE_PRIORITY="1")
        hp = subprocess.run([str(FAKE_DIR / "loop_app"), "--role", "hp", "--count", "8", "--log", str(tmp_path / "hp.log")], capture_output=True, text=True,
                            timeout=120, env=hp_env)
        assert hp.returncode == 0 and "DONE" in hp.stdout, hp.stdout + hp.stderr[-2000:]
        out, _ = lp.communicate(timeout=120)
        assert lp.returncode == 0, out
    finally:
        if lp is not None and lp.poll() is None:
            lp.kill()
        server.send_signal(signal.SIGTERM)
        server.wait(timeout=10)
    res = json.loads(out.strip().splitlines()[-1])
    assert res["finished"] == res["expected"] == 90 and res["bad_tiles"] == 0, res
    assert res["deactivations"] >= 4 and res["relaunches"] >= res["preemptions"] >= 1, res


@pytest.mark.parametrize("sanitizer", ["thread", "address,undefined"])
def test_interposer_and_hal_are_clean_under_sanitizers(tmp_path, sanitizer):
    """Everything between the program and the fake driver — interposer, CUDA HAL, XQueue runtime, scheduler —
    compiled with ThreadSanitizer, then with AddressSanitizer + UBSan (the driver is opened without RTLD_DEEPBIND
    in such builds; leak checking is off: the process-lifetime singletons are never freed by design)."""
    srcs = [CSRC / "shim" / "shim.cpp"] + [p for d in ("hal_cuda", "preempt", "sched", "utils") for p in sorted((CSRC / d).glob("*.cpp"))]
    common = [CXX, "-O1", "-g", f"-fsanitize={sanitizer}", "-fno-omit-frame-pointer", "-fPIC", "-pthread", f"-I{ROOT / 'include'}", f"-I{CSRC}", f"-I{CUDA_INC}"]
    san_env = dict(TSAN_OPTIONS="halt_on_error=0", ASAN_OPTIONS="detect_leaks=0")
    markers = ("WARNING: ThreadSanitizer", "ERROR: AddressSanitizer", "runtime error:")

    def clean(text: str) -> bool:
        return not any(m in text for m in markers)

    def compile_one(src: Path):
        obj = tmp_path / (src.parent.name + "_" + src.stem + ".o")
        r = subprocess.run(common + ["-std=c++20", "-DXSCHED_NO_DEEPBIND", "-c", "-o", str(obj), str(src)], capture_output=True, text=True)
        return obj, r
    with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as pool:
        objs = []
        for obj, r in pool.map(compile_one, srcs):
            assert r.returncode == 0, r.stderr[-2000:]
            objs.append(str(obj))
    shim = tmp_path / "libshim_tsan.so"
    r = subprocess.run(common + ["-shared", "-Wl,-soname,libcuda.so.1", "-o", str(shim)] + objs + [f"-L{LIB}", f"-Wl,-rpath,{LIB}", "-lxpk", "-ldl", "-lrt"],
                       capture_output=True, text=True)
    if r.returncode != 0 and ("cannot find" in r.stderr or "unrecognized" in r.stderr):
        pytest.skip(f"toolchain has no -fsanitize={sanitizer} runtime")
    assert r.returncode == 0, r.stderr[-2000:]
    fake, app = tmp_path / "libcuda_fake_tsan.so", tmp_path / "driver_app_tsan"
    for cmd in (common + ["-std=c++17", "-shared", "-Wl,-soname,libcuda.so.1", "-o", str(fake), str(FAKE_DIR / "fake_cuda.cpp"), "-ldl"],
                common + ["-std=c++17", "-o", str(app), str(FAKE_DIR / "driver_app.cpp"), f"-L{FAKE_DIR / 'link'}", "-lcuda", "-ldl"]):
        r = subprocess.run(cmd, capture_output=True, text=True)
        assert r.returncode == 0, r.stderr[-2000:]
    # the XSched-aware program: the same objects without the interposer in front
    hal_tsan = tmp_path / "hal_app_tsan"
    no_shim = [o for o in objs if not o.endswith("shim_shim.o")]
    r = subprocess.run(common + ["-std=c++17", f"-I{ROOT / 'include'}", "-o", str(hal_tsan), str(FAKE_DIR / "hal_app.cpp")] + no_shim +
                       [f"-L{FAKE_DIR / 'link'}", f"-L{LIB}", f"-Wl,-rpath,{LIB}", "-lxpk", "-lcuda", "-ldl", "-lrt"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    r = run_app(as_libcuda(tmp_path, fake), fake, hal_tsan, XSCHED_CUDA_LIB=fake, **san_env)
    text = r.stdout + r.stderr
    assert clean(text), text[-4000:]
    assert r.returncode == 0, text[-2000:]
    # level 2 with fake preemptible tasks (fake_xpk.cpp instead of libxpk)
    l2_tsan = tmp_path / "level2_app_tsan"
    r = subprocess.run(common + ["-std=c++20", f"-I{ROOT / 'include'}", "-o", str(l2_tsan), str(FAKE_DIR / "level2_app.cpp"), str(FAKE_DIR / "fake_xpk.cpp")] +
                       no_shim + [f"-L{FAKE_DIR / 'link'}", "-lcuda", "-ldl", "-lrt"], capture_output=True, text=True)
    assert r.returncode == 0, r.stderr[-2000:]
    r = run_app(as_libcuda(tmp_path, fake), fake, l2_tsan, XSCHED_CUDA_LIB=fake, **san_env)
    text = r.stdout + r.stderr
    assert clean(text), text[-4000:]
    assert r.returncode == 0 and '"bad_tiles": 0' in r.stdout, text[-2000:]
    for level in (1, 2):
        r = run_app(as_libcuda(tmp_path, shim), fake, app, XSCHED_CUDA_LIB=fake, XSCHED_AUTO_XQUEUE="ON", XSCHED_POLICY="HPF",
                    XSCHED_AUTO_XQUEUE_LEVEL=level, XSCHED_AUTO_XQUEUE_THRESHOLD=4, XSCHED_AUTO_XQUEUE_BATCH_SIZE=2, **san_env)
        text = r.stdout + r.stderr
        assert clean(text), text[-4000:]
        assert r.returncode == 0 and r.stdout.startswith("OK "), text[-2000:]


@pytest.mark.parametrize("spin,level", [("OFF", 1), ("ON", 1), ("OFF", 2)])
def test_transparent_two_process_scheduling_without_a_gpu(tmp_path, spin, level):
    """Two XSched-unaware processes under the interposer, one xserver (HPF), priorities 0 and 1 from the
    environment — the reference's transparent mode, end to end on the fake driver: while the high-priority
    process has a request in flight the low-priority process's stream must stand still (after the at most
    `threshold` kernels already handed to the driver have drained: ordinary kernels cannot be deactivated, so
    level 2 behaves like level 1 for them, but the queue's Deactivate / Reactivate path runs)."""
    import signal
    import time
    loop_app = FAKE_DIR / "loop_app"
    assert loop_app.exists(), "tests/fake_cuda/loop_app not built (python -m xsched_b200.build)"
    ns = f"fk{os.getpid()}{spin}{level}."
    libdir = as_libcuda(tmp_path, LIB / "libshimcuda.so")
    base = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
    base.update(FAKE_CUDA_LIB=str(FAKE), XSCHED_CUDA_LIB=str(FAKE), LD_LIBRARY_PATH=f"{libdir}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""),
                XLOG_LEVEL="WARN", XSCHED_IPC_NAMESPACE=ns, XSCHED_IPC_SPIN=spin, XSCHED_SCHEDULER="GLB", XSCHED_AUTO_XQUEUE="ON",
                XSCHED_AUTO_XQUEUE_LEVEL=str(level), XSCHED_AUTO_XQUEUE_THRESHOLD="4", XSCHED_AUTO_XQUEUE_BATCH_SIZE="2")
    srv_env = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
    srv_env.update(XSCHED_IPC_NAMESPACE=ns, XSCHED_IPC_SPIN=spin, XLOG_LEVEL="WARN")
    server = subprocess.Popen([str(LIB / "xserver"), "HPF", "50000"], stdout=subprocess.PIPE, text=True, env=srv_env)
    lp = None
    try:
        assert "ready" in server.stdout.readline()
        lp_log, hp_log = tmp_path / "lp.log", tmp_path / "hp.log"
        lp = subprocess.Popen([str(loop_app), "--role", "lp", "--log", str(lp_log)], stdout=subprocess.PIPE, text=True,
                              env=dict(base, XSCHED_AUTO_XQUEUE_PRIORITY="0"))
        assert lp.stdout.readline().startswith("READY")
        time.sleep(0.1)
        hp = subprocess.run([str(loop_app), "--role", "hp", "--count", "6", "--log", str(hp_log)], capture_output=True, text=True, timeout=120,
                            env=dict(base, XSCHED_AUTO_XQUEUE_PRIORITY="1"))
        assert hp.returncode == 0 and "DONE" in hp.stdout, hp.stdout + hp.stderr[-2000:]
        time.sleep(0.1)
    finally:
        if lp is not None:
            lp.send_signal(signal.SIGTERM)
            lp.communicate(timeout=60)
        server.send_signal(signal.SIGTERM)
        server.wait(timeout=10)
    starts = [int(x) for x in lp_log.read_text().split()]
    requests = [tuple(map(int, line.split())) for line in hp_log.read_text().splitlines()]
    assert len(requests) == 6 and len(starts) > 100
    for t0, t1 in requests:
        assert t1 - t0 >= 40 * 300
        # grace = the first half of the request: the ready event has to reach the server and the suspend the other
        # process (on a busy test host a polling thread can lose its core for milliseconds), then up to four
        # kernels that were already with the driver finish
        inside = [t for t in starts if t0 + (t1 - t0) // 2 < t < t1 - 200]
        # Unsuspended, the other process would start about (t1 - t0) / 2 / 350 us kernels here.  A handful is
        # tolerated: when the requesting thread loses its core in the middle of its burst, its queue drains, the
        # low-priority queue is rightly resumed for a moment and suspended again.
        allowed = max(4, (t1 - t0) // 2 // 350 // 10)
        assert len(inside) <= allowed, f"low-priority kernels started {len(inside)} times inside a high-priority request of {t1 - t0} us"
    # and it does run between the requests
    gaps = [(requests[i][1], requests[i + 1][0]) for i in range(len(requests) - 1)]
    assert all(sum(1 for t in starts if a + 3000 < t < b) > 3 for a, b in gaps)


PTDS_APP = FAKE_DIR / "ptds_app"


def run_ptds(libdir: Path, *args, **extra):
    env = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
    env.update(FAKE_CUDA_LIB=str(FAKE), LD_LIBRARY_PATH=f"{libdir}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""), XLOG_LEVEL="WARN")
    env.update({k: str(v) for k, v in extra.items()})
    return subprocess.run([str(PTDS_APP), *map(str, args)], capture_output=True, text=True, env=env, timeout=300)


def test_per_thread_default_stream_is_scheduled(tmp_path):
    """CU_STREAM_PER_THREAD and the `_ptsz` entry points (looked up with the per-thread flag): every thread's default
    stream becomes a private stream with an XQueue; nothing bypasses the queues; same results as without the interposer."""
    plain = run_ptds(as_libcuda(tmp_path, FAKE), 3, 20)
    assert plain.returncode == 0 and plain.stdout.startswith("OK "), plain.stdout + plain.stderr
    stats = tmp_path / "stats.json"
    r = run_ptds(as_libcuda(tmp_path, LIB / "libshimcuda.so"), 3, 20, XSCHED_CUDA_LIB=FAKE, XSCHED_AUTO_XQUEUE="ON", XSCHED_POLICY="HPF",
                 XSCHED_AUTO_XQUEUE_LEVEL=1, XSCHED_AUTO_XQUEUE_THRESHOLD=4, XSCHED_AUTO_XQUEUE_BATCH_SIZE=2, XSCHED_SHIM_STATS_FILE=stats)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert r.stdout == plain.stdout
    st = json.loads(stats.read_text())
    assert st["thread_streams"] == 3 and st["streams_with_xqueue"] == 3
    assert st["launches_queued"] == 3 * 20 * 2 and st["launches_direct"] == 0
    assert st["copies_queued"] == 3 * 20 * 2 and st["copies_direct"] == 0
    assert st["syncs_via_xqueue"] == 3 * 20
    assert st["getproc_hooked_ptsz"] == 3 * 5            # five per-thread lookups per thread, all answered with the twins


def test_single_stream_per_process(tmp_path):
    """XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS=ON: four stream creations hand out one reference-counted stream; work
    given to any handle is ordered (the program's kernels on four handles read and write the same buffer, which is
    only correct when the handles are one stream); the stream lives until its last handle is destroyed."""
    stats = tmp_path / "stats.json"
    r = run_ptds(as_libcuda(tmp_path, LIB / "libshimcuda.so"), 1, 9, "single", XSCHED_CUDA_LIB=FAKE, XSCHED_AUTO_XQUEUE="ON", XSCHED_POLICY="HPF",
                 XSCHED_AUTO_XQUEUE_LEVEL=1, XSCHED_CUDA_SINGLE_STREAM_PER_PROCESS="ON", XSCHED_SHIM_STATS_FILE=stats)
    assert r.returncode == 0, r.stdout + r.stderr[-3000:]
    assert r.stdout.startswith("OK 136 same_handles=1")
    st = json.loads(stats.read_text())
    assert st["single_stream_refs"] == 4 and st["streams_with_xqueue"] == 1 and st["launches_queued"] == 9


def test_transfer_aware_readiness_keeps_lower_priorities_running_during_copies(tmp_path):
    """XSCHED_TRANSFER_AWARE_READY=ON (an addition, off by default): a high-priority request that is copy-in, one
    kernel, copy-out only takes the "device" away from the low-priority queue for about the kernel's time; with the
    reference's readiness rule (a queue is ready while anything is queued) the copies count as well."""
    app = FAKE_DIR / "transfer_app"
    assert app.exists()
    out = {}
    for mode in ("OFF", "ON"):
        env = {k: v for k, v in os.environ.items() if not k.startswith("XSCHED_")}
        env.update(FAKE_CUDA_LIB=str(FAKE), XSCHED_CUDA_LIB=str(FAKE), XLOG_LEVEL="WARN", XSCHED_TRANSFER_AWARE_READY=mode,
                   LD_LIBRARY_PATH=f"{as_libcuda(tmp_path, FAKE)}:{LIB}:" + os.environ.get("LD_LIBRARY_PATH", ""))
        r = subprocess.run([str(app), "4"], capture_output=True, text=True, env=env, timeout=120)
        assert r.returncode == 0 and r.stdout.startswith("{"), r.stdout + r.stderr[-2000:]
        out[mode] = json.loads(r.stdout)
    on, off = out["ON"], out["OFF"]
    assert off["lp_held_back_us"] > 3 * off["hp_kernel_us"]            # the copies kept the low-priority queue out
    assert on["lp_held_back_us"] < 2.5 * on["hp_kernel_us"]            # about the kernels' time only
    assert on["lp_kernels"] > 2 * off["lp_kernels"]
