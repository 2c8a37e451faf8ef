"""High-priority workload generator: batch-1 decode on a random-init Llama-3-8B-shaped model in bf16
(32 layers, hidden 4096, 32 query / 8 KV heads of 128, FFN 14336, KV length 4096, vocabulary 128256 assumed),
requests of N tokens arriving as a Poisson process.  Pure PyTorch (library kernels): this is a WORKLOAD for the
scheduler, not part of the preemption path — it is meant to be run unchanged under the libcuda interposer,

    LD_LIBRARY_PATH=<dir with libcuda.so.1 -> libshimcuda.so>  XSCHED_AUTO_XQUEUE=ON XSCHED_SCHEDULER=GLB \
    XSCHED_AUTO_XQUEUE_PRIORITY=1  python -m xsched_b200.llama_decode --requests 20 --rate 2

so that its stream becomes a high-priority XQueue.  Weights are synthetic (seeded normal, std 0.02); no
checkpoint or dataset is involved.  Prints one JSON line with per-token and per-request latency percentiles.
Each decode step reads every weight once (~15.0 GB) plus the KV cache (~0.54 GB): HBM-bound, ~2.4 ms at the
measured 6.5 TB/s.

With --batched the requests in flight are decoded together (continuous batching: one step streams the weights once
for all of them, every request is still a batch-1 client with its own KV cache of 4096 positions and its own 128
tokens).  That is what makes the configured 10 requests/s servable at all: one request at a time needs ~0.7 s of
decode per request, seven times more than one GPU has at that rate.  A token's latency is then the duration of the
step that produced it, counted once per request that was in the step.
"""
from __future__ import annotations

import argparse
import json
import random
import time

import torch

H, NQ, NKV, HD, FFN, LAYERS, VOCAB = 4096, 32, 8, 128, 14336, 32, 128256


def pct(v, p):
    v = sorted(v)
    return v[min(len(v) - 1, int(p * (len(v) - 1) + 0.5))] if v else float("nan")


class Layer:
    def __init__(self, g, kv_len, dev, slots=1):
        def w(o, i):
            return (torch.randn(o, i, device=dev, generator=g, dtype=torch.float32) * 0.02).to(torch.bfloat16)
        self.wqkv = w((NQ + 2 * NKV) * HD, H)
        self.wo = w(H, NQ * HD)
        self.w_gate_up = w(2 * FFN, H)
        self.w_down = w(H, FFN)
        self.n1 = torch.ones(H, device=dev, dtype=torch.bfloat16)
        self.n2 = torch.ones(H, device=dev, dtype=torch.bfloat16)
        self.k = (torch.randn(1, NKV, kv_len, HD, device=dev, generator=g) * 0.5).to(torch.bfloat16).expand(slots, -1, -1, -1).contiguous()
        self.v = (torch.randn(1, NKV, kv_len, HD, device=dev, generator=g) * 0.5).to(torch.bfloat16).expand(slots, -1, -1, -1).contiguous()

    def __call__(self, x, pos):
        h = torch.nn.functional.rms_norm(x, (H,), self.n1, 1e-5)
        qkv = h @ self.wqkv.T
        q, k, v = qkv.split([NQ * HD, NKV * HD, NKV * HD], dim=-1)
        # the new token's K/V overwrite one cache slot (fixed KV length: a sliding window of 4096)
        self.k[0, :, pos] = k.view(NKV, HD)
        self.v[0, :, pos] = v.view(NKV, HD)
        att = torch.nn.functional.scaled_dot_product_attention(q.view(1, NQ, 1, HD), self.k, self.v, enable_gqa=True)
        x = x + att.reshape(1, NQ * HD) @ self.wo.T
        h = torch.nn.functional.rms_norm(x, (H,), self.n2, 1e-5)
        gu = h @ self.w_gate_up.T
        g_, u_ = gu.split([FFN, FFN], dim=-1)
        return x + (torch.nn.functional.silu(g_) * u_) @ self.w_down.T

    def batched(self, x, rows, pos):
        """n requests at once: x [n, H], rows = arange(n) (their cache slots), pos [n] = each one's write position."""
        n = x.shape[0]
        h = torch.nn.functional.rms_norm(x, (H,), self.n1, 1e-5)
        qkv = h @ self.wqkv.T
        q, k, v = qkv.split([NQ * HD, NKV * HD, NKV * HD], dim=-1)
        self.k[rows, :, pos] = k.view(n, NKV, HD)
        self.v[rows, :, pos] = v.view(n, NKV, HD)
        att = torch.nn.functional.scaled_dot_product_attention(q.view(n, NQ, 1, HD), self.k[:n], self.v[:n], enable_gqa=True)
        x = x + att.reshape(n, NQ * HD) @ self.wo.T
        h = torch.nn.functional.rms_norm(x, (H,), self.n2, 1e-5)
        gu = h @ self.w_gate_up.T
        g_, u_ = gu.split([FFN, FFN], dim=-1)
        return x + (torch.nn.functional.silu(g_) * u_) @ self.w_down.T

    def move_slot(self, src, dst):
        """The request in cache slot `src` continues in slot `dst` (slots in use stay contiguous)."""
        self.k[dst].copy_(self.k[src])
        self.v[dst].copy_(self.v[src])


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--requests", type=int, default=20)
    ap.add_argument("--tokens", type=int, default=128)
    ap.add_argument("--rate", type=float, default=10.0, help="mean request arrivals per second (Poisson)")
    ap.add_argument("--kv", type=int, default=4096)
    ap.add_argument("--layers", type=int, default=LAYERS)
    ap.add_argument("--seed", type=int, default=7)
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--deadline-ms", type=float, default=0.0, help="count decode steps that took longer than this (0 = off)")
    ap.add_argument("--samples", default="", help="write every per-token latency (ms, one per line) to this file")
    ap.add_argument("--batched", action="store_true", help="decode the requests in flight together (continuous batching)")
    ap.add_argument("--max-batch", type=int, default=16)
    a = ap.parse_args()
    torch.cuda.set_device(a.device)
    dev = torch.device("cuda", a.device)
    g = torch.Generator(device=dev).manual_seed(a.seed)
    layers = [Layer(g, a.kv, dev, a.max_batch if a.batched else 1) for _ in range(a.layers)]
    lm_head = (torch.randn(VOCAB, H, device=dev, generator=g) * 0.02).to(torch.bfloat16)
    norm = torch.ones(H, device=dev, dtype=torch.bfloat16)
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()          # created after the interposer is in place: gets its own XQueue
    rng = random.Random(a.seed)

    def step(x, pos):
        for l in layers:
            x = l(x, pos)
        logits = torch.nn.functional.rms_norm(x, (H,), norm, 1e-5) @ lm_head.T
        return x, int(logits.argmax())          # the .item() is the device->host read of the step's result

    tok_ms, req_ms = [], []
    batch_sizes = []
    if a.batched:
        with torch.cuda.stream(stream), torch.no_grad():
            xb = torch.randn(a.max_batch, H, device=dev, generator=g).to(torch.bfloat16)
            rows_all = torch.arange(a.max_batch, device=dev)

            def bstep(n, pos_list):
                pos = torch.tensor(pos_list, device=dev)
                x = xb[:n]
                for l in layers:
                    x = l.batched(x, rows_all[:n], pos)
                xb[:n] = x
                logits = torch.nn.functional.rms_norm(x, (H,), norm, 1e-5) @ lm_head.T
                return logits.argmax(dim=-1).tolist()      # the device->host read of the step's result

            for n in list(range(1, a.max_batch + 1)) * 2:                      # warm-up: every batch size once picks its kernels
                bstep(n, [n] * n)
            print("READY", flush=True)
            t0 = time.perf_counter()
            arrivals, t = [], t0
            for _ in range(a.requests):
                t += rng.expovariate(a.rate)
                arrivals.append(t)
            active = []                               # [arrival time, tokens done, write position]; index = cache slot
            nxt = 0
            while nxt < len(arrivals) or active:
                now = time.perf_counter()
                while nxt < len(arrivals) and arrivals[nxt] <= now and len(active) < a.max_batch:
                    active.append([arrivals[nxt], 0, (nxt * 37) % a.kv])
                    nxt += 1
                if not active:
                    time.sleep(max(0.0, arrivals[nxt] - time.perf_counter()))
                    continue
                n = len(active)
                ts = time.perf_counter()
                bstep(n, [r[2] for r in active])
                dt = (time.perf_counter() - ts) * 1e3
                tok_ms.extend([dt] * n)
                batch_sizes.append(n)
                end = time.perf_counter()
                slot = 0
                while slot < len(active):
                    r = active[slot]
                    r[1] += 1
                    r[2] = (r[2] + 1) % a.kv
                    if r[1] < a.tokens:
                        slot += 1
                        continue
                    req_ms.append((end - r[0]) * 1e3)
                    last = len(active) - 1
                    if slot != last:                  # the last slot's request moves into the freed one
                        for l in layers:
                            l.move_slot(last, slot)
                        xb[slot].copy_(xb[last])
                        active[slot] = active[last]
                    active.pop()
    if not a.batched:
        with torch.cuda.stream(stream), torch.no_grad():
            x = torch.randn(1, H, device=dev, generator=g).to(torch.bfloat16)
            for i in range(3):
                x, _ = step(x, i)                    # warm-up (cuBLAS heuristics, allocator)
            print("READY", flush=True)
            t_next = time.perf_counter()
            for r in range(a.requests):
                t_next += rng.expovariate(a.rate)
                now = time.perf_counter()
                if now < t_next:
                    time.sleep(t_next - now)
                t_arr = t_next                        # latency is counted from the arrival, queueing included
                for t in range(a.tokens):
                    t0 = time.perf_counter()
                    x, _ = step(x, (r * a.tokens + t) % a.kv)
                    tok_ms.append((time.perf_counter() - t0) * 1e3)
                req_ms.append((time.perf_counter() - t_arr) * 1e3)
    print("DONE", flush=True)
    if a.samples:
        with open(a.samples, "w") as f:
            f.write("\n".join(f"{v:.4f}" for v in tok_ms))
    missed = sum(1 for v in tok_ms if a.deadline_ms > 0 and v > a.deadline_ms)
    weights_gb = sum(p.numel() for l in layers for p in (l.wqkv, l.wo, l.w_gate_up, l.w_down)) * 2 / 1e9 + lm_head.numel() * 2 / 1e9
    print(json.dumps({"role": "llama-decode", "requests": len(req_ms), "tokens": len(tok_ms), "token_p50_ms": round(pct(tok_ms, 0.5), 3),
                      "token_p99_ms": round(pct(tok_ms, 0.99), 3), "token_mean_ms": round(sum(tok_ms) / max(1, len(tok_ms)), 3),
                      "request_p50_ms": round(pct(req_ms, 0.5), 2), "request_p99_ms": round(pct(req_ms, 0.99), 2),
                      "weights_gb": round(weights_gb, 2), "kv_gb": round(a.layers * 2 * NKV * a.kv * HD * 2 / 1e9, 3), "rate": a.rate,
                      "mode": "batched" if a.batched else "one request at a time", "decode_steps": len(batch_sizes) if a.batched else len(tok_ms),
                      "mean_batch": round(sum(batch_sizes) / max(1, len(batch_sizes)), 2) if a.batched else 1.0,
                      "deadline_ms": a.deadline_ms, "deadline_missed": missed, "deadline_miss_rate": round(missed / max(1, len(tok_ms)), 5)}))


if __name__ == "__main__":
    main()
