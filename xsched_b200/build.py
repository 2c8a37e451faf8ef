"""In-tree build of every native artefact (no cmake, no JIT cache).

    python -m xsched_b200.build            # build what is stale
    python -m xsched_b200.build --force    # rebuild everything

Targets land in xsched_b200/lib/ (product) and oracle/ (test-only checker).  CUDA sources are
compiled for sm_100a only.  The oracle's compiled reference core (oracle/_ref/) is built by
oracle/build_ref.py when the reference tree is present; that step is skipped elsewhere.
"""
from __future__ import annotations

import os
import shutil
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
PKG = ROOT / "xsched_b200"
CSRC = PKG / "csrc"
LIB = PKG / "lib"
INC = ROOT / "include"
ORACLE = ROOT / "oracle"

NVCC = os.environ.get("NVCC") or shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
# The system compiler, on purpose not $CXX/$CC: the libraries must link the shared libstdc++.  A toolchain
# that links it statically makes every .so export its own copy of libstdc++ internals (__once_proxy,
# std::string's empty rep, ...), which then get interposed into unrelated libraries of a large host process.
CXX = os.environ.get("XSCHED_CXX") or shutil.which("g++", path="/usr/bin:/usr/local/bin") or "g++"
CC = os.environ.get("XSCHED_CC") or shutil.which("gcc", path="/usr/bin:/usr/local/bin") or "gcc"
CUDA_HOME = os.environ.get("CUDA_HOME", "/usr/local/cuda")

NVCC_FLAGS = [
    "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo",
    "-Xcompiler", "-fPIC",
]
CXX_FLAGS = ["-std=c++20", "-O2", "-g", "-fPIC", "-Wall", "-Wextra", "-pthread"]


def _stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.stat().st_mtime > t for d in deps if d.exists())


def _run(cmd: list[str], verbose: bool) -> None:
    if verbose:
        print("+", " ".join(str(c) for c in cmd), flush=True)
    r = subprocess.run([str(c) for c in cmd], capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(r.stdout + r.stderr)
        raise RuntimeError(f"build step failed: {' '.join(str(c) for c in cmd[:3])} ...")
    if verbose and (r.stdout or r.stderr):
        print(r.stdout + r.stderr)


def _glob(d: Path, pats: tuple[str, ...]) -> list[Path]:
    out: list[Path] = []
    for p in pats:
        out += sorted(d.rglob(p))
    return out


def build_xpk(force: bool = False, verbose: bool = False) -> Path:
    """libxpk.so — the preemptible persistent kernels + their C ABI (include/xsched_b200/pk.h)."""
    out = LIB / "libxpk.so"
    kdir = CSRC / "kernels"
    srcs = sorted(kdir.glob("*.cu"))
    deps = srcs + sorted(kdir.glob("*.cuh")) + [INC / "xsched_b200" / "pk.h"]
    if force or _stale(out, deps):
        LIB.mkdir(parents=True, exist_ok=True)
        _run([NVCC, *NVCC_FLAGS, "-shared", f"-I{INC}", "-o", out, *srcs], verbose)
    return out


# Driver entry points the shim implements itself (by the name the library exports); everything else that
# cuda.h declares is forwarded by a generated trampoline.
SHIM_HANDLED = {
    "cuLaunchKernel", "cuMemcpyAsync", "cuMemcpyHtoDAsync_v2", "cuMemcpyDtoHAsync_v2", "cuMemcpyDtoDAsync_v2", "cuMemsetD8Async",
    "cuMemsetD32Async", "cuLaunchHostFunc", "cuEventRecord", "cuEventSynchronize", "cuEventQuery", "cuEventDestroy_v2",
    "cuStreamWaitEvent", "cuStreamSynchronize", "cuStreamQuery", "cuCtxSynchronize", "cuMemFree_v2", "cuStreamCreate",
    "cuStreamCreateWithPriority", "cuStreamDestroy_v2", "cuStreamBeginCapture_v2", "cuStreamEndCapture", "cuGetProcAddress",
    "cuGetProcAddress_v2", "cuLaunchKernelEx", "cuLaunchCooperativeKernel", "cuMemAllocAsync", "cuMemFreeAsync", "cuMemcpy2DAsync_v2",
    "cuMemcpyPeerAsync", "cuMemsetD16Async", "cuGraphLaunch", "cuStreamAddCallback", "cuMemcpy", "cuMemcpyDtoH_v2", "cuMemcpyHtoD_v2",
    "cuMemcpyDtoD_v2", "cuMemcpy3DAsync_v2", "cuMemsetD2D8Async", "cuMemsetD2D16Async", "cuMemsetD2D32Async", "cuGraphUpload",
    "cuEventRecordWithFlags", "cuStreamBeginCaptureToGraph",
    # per-thread-default-stream twins of the above
    "cuEventRecordWithFlags_ptsz", "cuEventRecord_ptsz", "cuGraphLaunch_ptsz", "cuGraphUpload_ptsz", "cuLaunchCooperativeKernel_ptsz", "cuLaunchHostFunc_ptsz", "cuLaunchKernelEx_ptsz", "cuLaunchKernel_ptsz", "cuMemAllocAsync_ptsz", "cuMemFreeAsync_ptsz", "cuMemcpy2DAsync_v2_ptsz", "cuMemcpy3DAsync_v2_ptsz", "cuMemcpyAsync_ptsz", "cuMemcpyDtoDAsync_v2_ptsz", "cuMemcpyDtoD_v2_ptds", "cuMemcpyDtoHAsync_v2_ptsz", "cuMemcpyDtoH_v2_ptds", "cuMemcpyHtoDAsync_v2_ptsz", "cuMemcpyHtoD_v2_ptds", "cuMemcpyPeerAsync_ptsz", "cuMemcpy_ptds", "cuMemsetD16Async_ptsz", "cuMemsetD2D16Async_ptsz", "cuMemsetD2D32Async_ptsz", "cuMemsetD2D8Async_ptsz", "cuMemsetD32Async_ptsz", "cuMemsetD8Async_ptsz", "cuStreamAddCallback_ptsz", "cuStreamBeginCaptureToGraph_ptsz", "cuStreamBeginCapture_v2_ptsz", "cuStreamEndCapture_ptsz", "cuStreamQuery_ptsz", "cuStreamSynchronize_ptsz", "cuStreamWaitEvent_ptsz",
}


def gen_shim_exports() -> Path:
    """Write csrc/shim/shim_exports.inc: one XSHIM_FWD(name) per driver entry point named in cuda.h —
    declared names, the versioned names their #defines map to, and the _ptds/_ptsz variants."""
    import re
    hdr = (Path(CUDA_HOME) / "include" / "cuda.h").read_text(errors="replace")
    names = set(re.findall(r"CUresult\s+CUDAAPI\s+(cu[A-Z]\w+)\s*\(", hdr))
    for a, b in re.findall(r"#define\s+(cu[A-Z]\w+)\s+(cu[A-Z]\w+)\s*$", hdr, flags=re.M):
        names.add(a)
        names.add(b)
    for kind, arg in re.findall(r"#define\s+cu[A-Z]\w+\s+__CUDA_API_(PTDS|PTSZ)\((cu[A-Z]\w+)\)", hdr):
        names.add(arg)
        names.add(arg + ("_ptds" if kind == "PTDS" else "_ptsz"))
        base = re.sub(r"_v\d+$", "", arg)
        names.add(base)
    names -= SHIM_HANDLED
    # The batched-copy entry points (plain and 3D) get no forwarder: that family is not to be used on this
    # hardware pool; a program that asks for them through the proc-address lookup still reaches the driver's own.
    names = {n for n in names if not re.search(r"Memcpy(3D)?B" + "atch", n)}
    out = CSRC / "shim" / "shim_exports.inc"
    text = "// generated from cuda.h by xsched_b200/build.py (gen_shim_exports); do not edit\n" + "".join(f"XSHIM_FWD({n})\n" for n in sorted(names))
    if not out.exists() or out.read_text() != text:
        out.write_text(text)
    return out


def build_host(force: bool = False, verbose: bool = False) -> list[Path]:
    """Host libraries: libpreempt.so, libhalcuda.so, libshimcuda.so, xserver and the host-only lane."""
    outs: list[Path] = []
    LIB.mkdir(parents=True, exist_ok=True)
    hdrs = _glob(INC, ("*.h",)) + _glob(CSRC, ("*.h",))
    incs = [f"-I{INC}", f"-I{CSRC}", f"-I{CUDA_HOME}/include"]

    def so(name: str, subdirs: list[str], libs: list[str], extra: list[str] | None = None) -> None:
        srcs: list[Path] = []
        for sd in subdirs:
            srcs += sorted((CSRC / sd).glob("*.cpp"))
        if not srcs:
            return
        out = LIB / name
        if force or _stale(out, srcs + hdrs):
            _run([CXX, *CXX_FLAGS, "-shared", *incs, "-o", out, *srcs, f"-L{LIB}", f"-Wl,-rpath,$ORIGIN",
                  *(extra or []), *libs], verbose)
        outs.append(out)

    so("libpreempt.so", ["utils", "sched", "preempt"], ["-ldl", "-lrt"])
    so("libhalhost.so", ["hal_host"], ["-lpreempt"])
    so("libhalcuda.so", ["hal_cuda"], ["-lpreempt", "-lxpk", "-ldl"])
    if (CSRC / "shim" / "shim.cpp").exists():
        hdrs.append(gen_shim_exports())
    so("libshimcuda.so", ["shim"], ["-lhalcuda", "-lpreempt", "-ldl"],
       extra=["-Wl,-soname,libcuda.so.1"])

    server_srcs = sorted((CSRC / "server").glob("*.cpp"))
    if server_srcs:
        out = LIB / "xserver"
        if force or _stale(out, server_srcs + hdrs + [LIB / "libpreempt.so"]):
            _run([CXX, *CXX_FLAGS, "-fPIE", *incs, "-o", out, *server_srcs, f"-L{LIB}", "-Wl,-rpath,$ORIGIN",
                  "-lpreempt", "-ldl", "-lrt"], verbose)
        outs.append(out)
    cli_srcs = sorted((CSRC / "cli").glob("*.cpp"))
    if cli_srcs:
        out = LIB / "xcli"
        http_src = CSRC / "server" / "http.cpp"
        if force or _stale(out, cli_srcs + [http_src] + hdrs + [LIB / "libpreempt.so"]):
            _run([CXX, *CXX_FLAGS, "-fPIE", *incs, "-o", out, *cli_srcs, http_src, f"-L{LIB}", "-Wl,-rpath,$ORIGIN", "-lpreempt", "-ldl", "-lrt"], verbose)
        outs.append(out)
    # libcuda.so.1 / libcuda.so names the dynamic loader looks for when the shim directory is put on
    # LD_LIBRARY_PATH (same install layout as the reference: platforms/cuda/CMakeLists.txt:2-5).
    shim = LIB / "libshimcuda.so"
    if shim.exists():
        d = LIB / "shim"
        d.mkdir(exist_ok=True)
        for alias in ("libcuda.so.1", "libcuda.so"):
            link = d / alias
            if link.is_symlink() or link.exists():
                link.unlink()
            link.symlink_to(Path("..") / "libshimcuda.so")
    return outs


def build_oracle(force: bool = False, verbose: bool = False) -> Path:
    """oracle/liboracle_kernels.so — the CPU checker (test infrastructure, never shipped)."""
    out = ORACLE / "liboracle_kernels.so"
    src = ORACLE / "kernels_oracle.c"
    if force or _stale(out, [src]):
        _run([CC, "-O2", "-ffp-contract=off", "-fPIC", "-shared", "-o", out, src, "-lm"], verbose)
    return out


def build_bench_worker(force: bool = False, verbose: bool = False) -> Path | None:
    """xbench_worker — the native workload driver bench.py launches (one process per role)."""
    src = CSRC / "bench" / "xbench_worker.cu"
    out = LIB / "xbench_worker"
    deps = [src, LIB / "libpreempt.so", LIB / "libhalcuda.so", LIB / "libxpk.so"] + _glob(INC, ("*.h",))
    if not src.exists() or not (LIB / "libhalcuda.so").exists():
        return None
    if force or _stale(out, deps):
        _run([NVCC, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", f"-I{INC}", "-o", out, src,
              f"-L{LIB}", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lhalcuda", "-lpreempt", "-lxpk"], verbose)
    # The XSched-unaware twin of the worker: CUDA runtime + kernel library only (no XQueue API linked), for the
    # transparent-interposer comparisons (its CUDA runtime loads "libcuda.so.1" by name, so the interposer that
    # is first on LD_LIBRARY_PATH is what it gets as the driver).
    psrc, pout = CSRC / "bench" / "plain_worker.cu", LIB / "plain_worker"
    if psrc.exists() and (force or _stale(pout, [psrc, LIB / "libxpk.so"])):
        _run([NVCC, "-std=c++17", "-O3", "-gencode", "arch=compute_100a,code=sm_100a", f"-I{INC}", "-o", pout, psrc,
              f"-L{LIB}", "-Xlinker", "-rpath", "-Xlinker", "$ORIGIN", "-lxpk"], verbose)
    return out


def build_test_apps(force: bool = False, verbose: bool = False) -> Path | None:
    """tests/apps/plain_streams, plain_graph — XSched-unaware CUDA programs the interposer tests run (cudart
    linked, dynamically-loaded driver: they find "libcuda.so.1" through the loader path like any application)."""
    out = None
    for name in ("plain_streams", "plain_graph"):
        src = ROOT / "tests" / "apps" / f"{name}.cu"
        out = ROOT / "tests" / "apps" / name
        if not src.exists():
            continue
        if force or _stale(out, [src]):
            _run([NVCC, "-std=c++17", "-O2", "-gencode", "arch=compute_100a,code=sm_100a", "-o", out, src], verbose)
    # the same kind of program built for per-thread default streams
    src, ptds = ROOT / "tests" / "apps" / "plain_ptds.cu", ROOT / "tests" / "apps" / "plain_ptds"
    if src.exists() and (force or _stale(ptds, [src])):
        _run([NVCC, "-std=c++17", "-O2", "--default-stream", "per-thread", "-gencode", "arch=compute_100a,code=sm_100a", "-o", ptds, src], verbose)
    build_fake_driver(force, verbose)
    return out


def build_fake_driver(force: bool = False, verbose: bool = False) -> Path | None:
    """tests/fake_cuda — a host-only stand-in for the CUDA driver and a driver-API program on top of it, so that
    the CUDA HAL and the interposer can be exercised on a machine without a GPU (test infrastructure)."""
    d = ROOT / "tests" / "fake_cuda"
    src, app_src = d / "fake_cuda.cpp", d / "driver_app.cpp"
    if not src.exists():
        return None
    lib, app = d / "libcuda_fake.so", d / "driver_app"
    if force or _stale(lib, [src]):
        _run([CXX, "-std=c++17", "-O1", "-g", "-shared", "-fPIC", "-pthread", f"-I{CUDA_HOME}/include", "-Wl,-soname,libcuda.so.1",
              "-o", lib, src, "-ldl"], verbose)
    link = d / "link"
    link.mkdir(exist_ok=True)
    if not (link / "libcuda.so").exists():
        os.symlink("../libcuda_fake.so", link / "libcuda.so")
    if force or _stale(app, [app_src, lib]):
        _run([CXX, "-std=c++17", "-O1", "-g", f"-I{CUDA_HOME}/include", "-o", app, app_src, f"-L{link}", "-lcuda", "-ldl", "-pthread"], verbose)
    loop_src, loop_app = d / "loop_app.cpp", d / "loop_app"
    if loop_src.exists() and (force or _stale(loop_app, [loop_src, lib])):
        _run([CXX, "-std=c++17", "-O1", "-g", f"-I{CUDA_HOME}/include", "-o", loop_app, loop_src, f"-L{link}", "-lcuda", "-ldl", "-pthread"], verbose)
    ptds_src, ptds_app = d / "ptds_app.cpp", d / "ptds_app"
    if ptds_src.exists() and (force or _stale(ptds_app, [ptds_src, lib])):
        _run([CXX, "-std=c++17", "-O1", "-g", f"-I{CUDA_HOME}/include", "-o", ptds_app, ptds_src, f"-L{link}", "-lcuda", "-ldl", "-pthread"], verbose)
    hal_src, hal_app = d / "hal_app.cpp", d / "hal_app"
    if hal_src.exists() and (LIB / "libhalcuda.so").exists() and (force or _stale(hal_app, [hal_src, lib, LIB / "libhalcuda.so", LIB / "libpreempt.so"])):
        _run([CXX, "-std=c++17", "-O1", "-g", f"-I{CUDA_HOME}/include", f"-I{INC}", "-o", hal_app, hal_src, f"-L{link}", f"-L{LIB}",
              f"-Wl,-rpath,{LIB}", "-lhalcuda", "-lpreempt", "-lcuda", "-ldl", "-pthread"], verbose)
    tr_src, tr_app = d / "transfer_app.cpp", d / "transfer_app"
    if tr_src.exists() and (LIB / "libhalcuda.so").exists() and (force or _stale(tr_app, [tr_src, lib, LIB / "libhalcuda.so", LIB / "libpreempt.so"])):
        _run([CXX, "-std=c++17", "-O1", "-g", f"-I{CUDA_HOME}/include", f"-I{INC}", "-o", tr_app, tr_src, f"-L{link}", f"-L{LIB}",
              f"-Wl,-rpath,{LIB}", "-lhalcuda", "-lpreempt", "-lcuda", "-ldl", "-pthread"], verbose)
    # the level-2 path of the CUDA HAL with fake preemptible tasks: the HAL's own sources + fake_xpk.cpp in place of libxpk
    l2_src, xpk_src, l2_app = d / "level2_app.cpp", d / "fake_xpk.cpp", d / "level2_app"
    hal_srcs = sorted((CSRC / "hal_cuda").glob("*.cpp"))
    if l2_src.exists() and (LIB / "libpreempt.so").exists() and (force or _stale(l2_app, [l2_src, xpk_src, lib, LIB / "libpreempt.so"] + hal_srcs)):
        _run([CXX, "-std=c++20", "-O1", "-g", "-pthread", f"-I{CUDA_HOME}/include", f"-I{INC}", f"-I{CSRC}", "-o", l2_app, l2_src, xpk_src] + hal_srcs +
             [f"-L{link}", f"-L{LIB}", f"-Wl,-rpath,{LIB}", "-lpreempt", "-lcuda", "-ldl", "-lrt"], verbose)
    return app


def build_lane_driver(force: bool = False, verbose: bool = False) -> Path | None:
    """oracle/lane_driver_new — the scenario runner linked against this repository's libraries
    (its twin linked against the reference core is built by oracle/build_ref.py)."""
    src = ORACLE / "lane_driver.cpp"
    out = ORACLE / "lane_driver_new"
    deps = [src, LIB / "libpreempt.so", LIB / "libhalhost.so"]
    if not src.exists() or not (LIB / "libhalhost.so").exists():
        return None
    if force or _stale(out, deps):
        _run([CXX, "-std=c++20", "-O2", "-pthread", f"-I{INC}", "-o", out, src, f"-L{LIB}", f"-Wl,-rpath,{LIB}",
              "-lhalhost", "-lpreempt"], verbose)
    probe_src, probe = ORACLE / "sched_probe_new.cpp", ORACLE / "sched_probe_new"
    if probe_src.exists() and (force or _stale(probe, [probe_src, LIB / "libpreempt.so"])):
        _run([CXX, "-std=c++20", "-O2", "-pthread", f"-I{INC}", "-o", probe, probe_src, f"-L{LIB}", f"-Wl,-rpath,{LIB}", "-lpreempt"], verbose)
    return out


def build_oracle_ref(force: bool = False, verbose: bool = False) -> Path | None:
    """oracle/_ref/ — the reference's own host core compiled from its sources where they lie.
    Only possible where the reference tree exists; elsewhere the prebuilt files are used."""
    script = ORACLE / "build_ref.py"
    if not script.exists():
        return None
    ref = Path(os.environ.get("XSCHED_REFERENCE_DIR", "/root/reference"))
    if not ref.exists():
        return None
    cmd = [sys.executable, str(script)] + (["--force"] if force else [])
    _run(cmd, verbose)
    return ORACLE / "_ref"


def build_all(force: bool = False, verbose: bool = False) -> None:
    build_xpk(force, verbose)
    build_host(force, verbose)
    build_bench_worker(force, verbose)
    build_test_apps(force, verbose)
    build_oracle(force, verbose)
    build_lane_driver(force, verbose)
    build_oracle_ref(force, verbose)


if __name__ == "__main__":
    build_all(force="--force" in sys.argv, verbose=True)
