# SPDX-License-Identifier: MIT
"""Device time of each kernel of one MMDiT block at the 12B shape (CUDA events,
L2 flushed between timed launches), with the achieved TFLOP/s or GB/s.

    python bench/mmdit/kernel_times.py [--tokens 4608] [--tp 1]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=4608)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--cublas", action="store_true", help="also time torch.matmul (cuBLAS) on the GEMM shapes")
    a = ap.parse_args()
    from barlink_sm86_b200 import ops
    dev = torch.device("cuda:0")
    H, heads, hd = 3072, 24 // a.tp, 128
    F = 4 * H // a.tp
    T = a.tokens
    g = torch.Generator(device=dev).manual_seed(0)
    rnd = lambda *s: (torch.randn(*s, generator=g, device=dev) * 0.05).bfloat16()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def timed(fn):
        for _ in range(3):
            fn()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            fn()
            e.record()
            torch.cuda.synchronize()
            ts.append(s.elapsed_time(e))
        ts.sort()
        return ts[len(ts) // 2] * 1e3  # us, median

    rows = []
    x = rnd(T, H)
    for name, n, k, kw in (("qkv", 3 * heads * hd, H, {}), ("proj", H, heads * hd, {}),
                           ("fc1+gelu", F, H, {"gelu": True}), ("fc2", H, F, {}),
                           ("single qkv", 3 * heads * hd, H, {}), ("single mlp+gelu", F, H, {"gelu": True})):
        w, b = rnd(n, k), rnd(n)
        xi = rnd(T, k)
        us = timed(lambda: ops.linear(xi, w, b, **kw))
        row = {"kernel": "linear " + name, "shape": [T, n, k], "us": us, "tflops": 2.0 * T * n * k / us / 1e6}
        if a.cublas:
            wt = w.t().contiguous()
            us2 = timed(lambda: torch.addmm(b, xi, wt))
            row["cublas_us"] = us2
        rows.append(row)
    qkv = rnd(T, 3 * heads * hd)
    v3 = qkv.unflatten(1, (3 * heads, hd))
    cu = torch.tensor([0, T], dtype=torch.int32, device=dev)
    us = timed(lambda: ops.attention(v3[:, :heads], v3[:, heads:2 * heads], v3[:, 2 * heads:], cu, cu, T,
                                     hd ** -0.5, False, max_k=T))
    rows.append({"kernel": "joint attention (V transpose + tcgen05)", "shape": [T, heads, hd], "us": us,
                 "tflops": 4.0 * T * T * heads * hd / us / 1e6})
    us = timed(lambda: ops.attention(v3[:, :heads], v3[:, heads:2 * heads], v3[:, 2 * heads:], cu, cu, T,
                                     hd ** -0.5, False))
    rows.append({"kernel": "joint attention (mma.sync)", "shape": [T, heads, hd], "us": us,
                 "tflops": 4.0 * T * T * heads * hd / us / 1e6})
    mod = rnd(1, 6 * H)
    gq = rnd(hd)
    pos = torch.zeros(T, 2, dtype=torch.int32, device=dev)
    us = timed(lambda: ops.layernorm_modulate(x, mod[:, :H], mod[:, H:2 * H], T))
    rows.append({"kernel": "layernorm_modulate", "us": us, "gbs": 2 * T * H * 2 / us / 1e3})
    us = timed(lambda: ops.qknorm_rope(qkv, gq, gq, pos, heads))
    rows.append({"kernel": "qknorm_rope", "us": us, "gbs": 2 * T * 2 * heads * hd * 2 / us / 1e3})
    y = rnd(T, H)
    us = timed(lambda: ops.gate_residual(x, y, mod[:, 2 * H:3 * H], T))
    rows.append({"kernel": "gate_residual", "us": us, "gbs": 3 * T * H * 2 / us / 1e3})
    for r in rows:
        print(json.dumps(r))


if __name__ == "__main__":
    main()
