"""Build the reference's own host core into oracle/_ref/ (TEST INFRASTRUCTURE, never shipped).

Compiles, from the sources where they lie in the reference tree (nothing is copied):
    utils/src/*.cpp  protocol/src/*.cpp  sched/src/*/*.cpp  preempt/src/*/*.cpp
with g++ -std=c++20 and the include roots  include/ utils/include protocol/include sched/include
preempt/include  plus oracle/stubs (the stand-in for the un-vendored `ipc` dependency), into
    oracle/_ref/libref_core.so
The reference's cmake build is not run.  Its CUDA HAL is NOT built here: it links the
un-vendored `cuxtra` library (driver-internal hooks) and cannot be reproduced.

On top of the core this script builds, against the REFERENCE headers, the host-only lane HAL and
the trace driver that tests and bench.py use to run the reference as the checker / CPU baseline:
    oracle/_ref/libhalhost_ref.so   from xsched_b200/csrc/hal_host/*.cpp
    oracle/_ref/lane_driver_ref     from oracle/lane_driver.cpp
    oracle/_ref/sched_probe_ref     from oracle/sched_probe_ref.cpp (drives the reference LocalScheduler + policies)
    oracle/_ref/libhalcuda_ref.so   the reference's CUDA HAL, level 1 only: platforms/cuda/hal/src/{common,level1}/*.cpp
                                    + oracle/stubs/cuda/arch_level1.cpp + oracle/stubs/cuxtra/cuxtra.h (stand-ins)
    oracle/_ref/libshimcuda_ref.so  the reference's libcuda interposer: platforms/cuda/shim/src/{shim,intercept}.cpp

Usage: python oracle/build_ref.py [--force]      (XSCHED_REFERENCE_DIR overrides the tree location)
"""
from __future__ import annotations

import os
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent
REF = Path(os.environ.get("XSCHED_REFERENCE_DIR", "/root/reference"))
OUT = HERE / "_ref"
OBJ = OUT / "obj"
import shutil
CXX = os.environ.get("XSCHED_CXX") or shutil.which("g++", path="/usr/bin:/usr/local/bin") or "g++"
FLAGS = ["-std=c++20", "-O2", "-fPIC", "-DRELEASE_MODE", "-pthread", "-w"]


def ref_includes() -> list[str]:
    return [f"-I{REF / d}" for d in ("include", "utils/include", "protocol/include", "sched/include", "preempt/include")] + \
           [f"-I{HERE / 'stubs'}"]


def run(cmd: list[str]) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    if r.returncode != 0:
        sys.stderr.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
        raise SystemExit(1)


def stale(out: Path, deps: list[Path]) -> bool:
    if not out.exists():
        return True
    t = out.stat().st_mtime
    return any(d.exists() and d.stat().st_mtime > t for d in deps)


def main() -> None:
    force = "--force" in sys.argv
    if not REF.exists():
        print(f"reference tree {REF} not present; keeping prebuilt oracle/_ref as is")
        return
    OBJ.mkdir(parents=True, exist_ok=True)
    srcs: list[Path] = []
    for pat in ("utils/src/*.cpp", "protocol/src/*.cpp", "sched/src/*/*.cpp", "preempt/src/*/*.cpp"):
        srcs += sorted(REF.glob(pat))
    core = OUT / "libref_core.so"
    stub = HERE / "stubs" / "ipc" / "ipc.h"
    if force or stale(core, srcs + [stub]):
        objs = []
        jobs = []
        for s in srcs:
            o = OBJ / (str(s.relative_to(REF)).replace("/", "_") + ".o")
            objs.append(o)
            jobs.append([CXX, *FLAGS, *ref_includes(), "-c", str(s), "-o", str(o)])
        with ThreadPoolExecutor(max_workers=os.cpu_count() or 4) as ex:
            list(ex.map(run, jobs))
        run([CXX, "-shared", "-o", str(core), *map(str, objs), "-lpthread", "-ldl"])
        print(f"built {core} from {len(srcs)} reference sources")

    link = [f"-L{OUT}", "-Wl,-rpath,$ORIGIN", "-lref_core", "-lpthread", "-ldl"]
    lane_srcs = sorted((ROOT / "xsched_b200" / "csrc" / "hal_host").glob("*.cpp"))
    lane_inc = f"-I{ROOT / 'xsched_b200' / 'csrc'}"
    lane = OUT / "libhalhost_ref.so"
    if lane_srcs and (force or stale(lane, lane_srcs + [core])):
        run([CXX, *FLAGS, *ref_includes(), lane_inc, "-shared", "-o", str(lane), *map(str, lane_srcs), *link])
        print(f"built {lane}")
    # ---- the reference's level-1 CUDA HAL and its libcuda shim (baseline "reference level 1 on this GPU") ----
    cuda = REF / "platforms" / "cuda"
    cuda_inc = [f"-I{cuda / 'hal' / 'include'}", f"-I{cuda / 'shim' / 'include'}"]
    hal_srcs = sorted((cuda / "hal" / "src" / "common").glob("*.cpp")) + sorted((cuda / "hal" / "src" / "level1").glob("*.cpp")) + \
        [HERE / "stubs" / "cuda" / "arch_level1.cpp"]
    hal = OUT / "libhalcuda_ref.so"
    if force or stale(hal, hal_srcs + [core, HERE / "stubs" / "cuxtra" / "cuxtra.h"]):
        run([CXX, *FLAGS, *ref_includes(), *cuda_inc, "-shared", "-o", str(hal), *map(str, hal_srcs), *link])
        print(f"built {hal} (reference sources: hal/src/common, hal/src/level1; stand-ins: cuxtra.h, arch_level1.cpp)")
    shim_srcs = [cuda / "shim" / "src" / "shim.cpp", cuda / "shim" / "src" / "intercept.cpp"]
    shim = OUT / "libshimcuda_ref.so"
    if force or stale(shim, shim_srcs + [hal]):
        run([CXX, *FLAGS, *ref_includes(), *cuda_inc, "-shared", "-Wl,-soname,libcuda.so.1", "-o", str(shim), *map(str, shim_srcs), *link,
             "-lhalcuda_ref"])
        print(f"built {shim}")
    shim_dir = OUT / "shim"
    shim_dir.mkdir(exist_ok=True)
    for alias in ("libcuda.so.1", "libcuda.so"):
        l = shim_dir / alias
        if l.is_symlink() or l.exists():
            l.unlink()
        l.symlink_to(Path("..") / "libshimcuda_ref.so")

    for name, srcname, extra in (("lane_driver", "lane_driver", ["-lhalhost_ref"]), ("sched_probe", "sched_probe_ref", [])):
        src = HERE / f"{srcname}.cpp"
        out = OUT / f"{name}_ref"
        if src.exists() and (force or stale(out, [src, core, lane])):
            run([CXX, *FLAGS, *ref_includes(), lane_inc, "-o", str(out), str(src), *link, *extra])
            print(f"built {out}")


if __name__ == "__main__":
    main()
