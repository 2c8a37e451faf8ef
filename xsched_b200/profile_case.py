"""Run a few launches of one preemptible kernel — the small, self-contained case used for ncu captures.

    python -m xsched_b200.profile_case gemm  [--m 8192 --n 8192 --k 8192] [--reps 3] [--flags 2]
    python -m xsched_b200.profile_case triad [--elems 268435456] [--reps 3] [--flags 0]
    python -m xsched_b200.profile_case sort  [--elems 16777216] [--reps 3]
    python -m xsched_b200.profile_case vecadd [--elems 67108864]

flags: 0 preemptible, 1 non-preemptible twin, 2 preemptible with in-flight abort (GEMM).
Prints the CUDA-event time of every launch.  Inputs are synthetic (seeded torch generators).
"""
from __future__ import annotations

import argparse

import torch

from . import pk


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("kernel", choices=["gemm", "triad", "sort", "vecadd"])
    ap.add_argument("--m", type=int, default=8192)
    ap.add_argument("--n", type=int, default=8192)
    ap.add_argument("--k", type=int, default=8192)
    ap.add_argument("--elems", type=int, default=0)
    ap.add_argument("--reps", type=int, default=3)
    ap.add_argument("--flags", type=int, default=0)
    ap.add_argument("--tile", type=int, default=0)
    a = ap.parse_args()
    torch.cuda.set_device(0)
    g = torch.Generator(device="cuda").manual_seed(1)
    s = torch.cuda.current_stream().cuda_stream
    restore = None
    if a.kernel == "gemm":
        x = torch.randn(a.m, a.k, device="cuda", generator=g).to(torch.bfloat16)
        y = torch.randn(a.n, a.k, device="cuda", generator=g).to(torch.bfloat16)
        z = torch.empty(a.m, a.n, device="cuda", dtype=torch.bfloat16)
        t = pk.Task.gemm(z, x, y, flags=a.flags)
        work, unit = 2.0 * a.m * a.n * a.k / 1e12, "TFLOP/s"
    elif a.kernel in ("triad", "vecadd"):
        n = a.elems or ((1 << 28) if a.kernel == "triad" else (1 << 26))
        x = torch.rand(n, device="cuda", generator=g) * 2 - 1
        y = torch.rand(n, device="cuda", generator=g) * 2 - 1
        z = torch.empty(n, device="cuda")
        t = pk.Task.triad(z, x, y, 1.5, tile_elems=a.tile, flags=a.flags) if a.kernel == "triad" else pk.Task.vecadd(z, x, y, tile_elems=a.tile, flags=a.flags)
        work, unit = 12.0 * n / 1e9, "GB/s"
    else:
        n = a.elems or (1 << 24)
        k0 = torch.randint(0, 2**31 - 1, (n,), dtype=torch.int32, device="cuda", generator=g)
        keys = k0.clone()
        tmp = torch.empty_like(keys)
        scratch = torch.empty(pk.sort_scratch_bytes(n), dtype=torch.uint8, device="cuda")
        t = pk.Task.sort(keys, tmp, scratch, flags=a.flags)
        restore = lambda: keys.copy_(k0)
        work, unit = 36.0 * n / 1e9, "GB/s"
    for i in range(a.reps):
        if restore:
            restore()
        t.reset(s)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        t.launch(s)
        e1.record()
        torch.cuda.synchronize()
        info = t.wait()
        ms = e0.elapsed_time(e1)
        print(f"{a.kernel} launch {i}: {ms:.4f} ms  {work / (ms * 1e-3):.1f} {unit}  status={info.status}")
    t.destroy()


if __name__ == "__main__":
    main()
