#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Decode linears of the Qwen2.5-7B shape inside a CUDA graph with rotating
weights (so that L2 does not hold them): the tcgen05 kernels against cuBLAS
(`F.linear`), and W8A16 against the bf16 kernel.  Reports time per call and the
weight-streaming bandwidth against the measured copy peak."""
import argparse
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200.ops import reference as ref  # noqa: E402


def graph_time(fn, ncalls, reps=5):
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for i in range(2):
            fn(i)
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for i in range(ncalls):
            fn(i)
    g.replay()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(reps):
        g.replay()
    e1.record()
    torch.cuda.synchronize()
    return e0.elapsed_time(e1) / reps / ncalls * 1e3


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    C = bl.load_extension()
    dev = torch.device("cuda", 0)
    peak = 6554.2
    try:
        peak = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))["hbm_gbs"]
    except Exception:
        pass
    H, I, V = 3584, 18944, 152064
    shapes = {"qkv": (4608, H), "o_proj": (H, H), "gate_up": (2 * I, H), "down": (H, I), "lm_head": (V, H)}
    rows = []
    for name, (n, k) in shapes.items():
        copies = max(2, int(600e6 // (n * k * 2)) + 1)
        ws = [torch.randn(n, k, device=dev, dtype=torch.bfloat16) * 0.02 for _ in range(copies)]
        x = torch.randn(args.batch, k, device=dev, dtype=torch.bfloat16)
        silu = name == "gate_up"
        calls = copies * 3
        t_mine = graph_time(lambda i: C.linear(x, ws[i % copies], None, None, silu), calls)
        t_slab = None
        if C.gemm_splits(n, k, args.batch) > 1:
            t_slab = graph_time(lambda i: C.linear_partial(x, ws[i % copies]), calls)
        t_lib = graph_time(lambda i: torch.nn.functional.linear(x, ws[i % copies]), calls)
        gb = n * k * 2 / 1e9
        row = dict(layer=name, n=n, k=k, tokens=args.batch, tcgen05_us=round(t_mine, 1),
                   tcgen05_slabs_us=round(t_slab, 1) if t_slab else None, cublas_us=round(t_lib, 1),
                   tcgen05_tbs=round(gb / (min(t_mine, t_slab or 1e9) * 1e-6) / 1e3, 2),
                   frac_of_measured_copy_peak=round(gb / (min(t_mine, t_slab or 1e9) * 1e-6) / peak, 3))
        wq = [ref.quantize_w8(w) for w in ws[:max(2, copies // 2)]]
        t_w8 = graph_time(lambda i: C.w8a16_linear(x, wq[i % len(wq)][0], wq[i % len(wq)][1]), len(wq) * 3)
        row["w8a16_us"] = round(t_w8, 1)
        row["w8a16_tbs"] = round(n * k / 1e9 / (t_w8 * 1e-6) / 1e3, 2)
        rows.append(row)
        print(row, flush=True)
        del ws, wq
    if args.out:
        json.dump(rows, open(args.out, "w"))


if __name__ == "__main__":
    main()
