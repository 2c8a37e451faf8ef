"""xsched_b200 — B200-native implementation of XSched's CUDA preemption path.

The package is a thin Python face over native libraries built in-tree under xsched_b200/lib/:

* libxpk.so       preemptible persistent sm_100a kernels (include/xsched_b200/pk.h)
* libpreempt.so   XQueue C API, HwQueue/HwCommand HAL contract, schedulers, HPF/LLF policies
* libhalcuda.so   CUDA HwQueue: Level-1 progressive launch window, Level-2 cooperative preemption
* libshimcuda.so  libcuda interposer
* xserver         the per-box scheduling server

There is no CPU fallback: importing a wrapper whose shared library is missing raises.
"""
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent
LIB_DIR = Path(__file__).resolve().parent / "lib"

__all__ = ["ROOT", "LIB_DIR"]
