#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""W8A16 decode GEMM: this library's tcgen05 kernel (bf16 activations, int8
per-channel weights widened in the main loop) against the reference's own
kernel pair built for sm_100 from baseline/_ref (`barlink_sm86._C.
w8a16_quant_act` + `w8a16_gemm`: int8 activations, dp4a, group-128 scales).
Shapes are the reference's decode shapes (torch_ext/tests/test_w8a16.py:23-32
there) plus the Qwen2.5-32B ones of the serving config."""
import importlib.util
import json
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200.ops import reference as ref  # noqa: E402
from bench.gemm.linear_bench import graph_time  # noqa: E402


def load_reference_ext():
    base = os.path.join(ROOT, "baseline", "_ref", "barlink_sm86")
    if not os.path.isdir(base):
        return None
    for f in sorted(os.listdir(base)):
        if f.startswith("_C") and f.endswith(".so"):
            spec = importlib.util.spec_from_file_location("barlink_sm86._C", os.path.join(base, f))
            mod = importlib.util.module_from_spec(spec)
            try:
                spec.loader.exec_module(mod)
                return mod
            except Exception as e:  # built against another torch, or no GPU
                print("reference extension did not load: %s" % e)
    return None


def main():
    C = bl.load_extension()
    R = load_reference_ext()
    dev = torch.device("cuda", 0)
    shapes = [(5120, 5120), (27648 * 2, 5120), (5120, 27648), (7168, 5120), (124160, 5120), (3072, 8704)]
    rows = []
    for m in (1, 4, 16, 64):
        for n, k in shapes:
            k128 = k // 128 * 128
            copies = max(2, int(300e6 // (n * k128)) + 1)
            w = [torch.randn(n, k128, device=dev) * 0.02 for _ in range(copies)]
            q = [ref.quantize_w8(t) for t in w]
            x = torch.randn(m, k128, device=dev).to(torch.bfloat16)
            t_mine = graph_time(lambda i: C.w8a16_linear(x, q[i % copies][0], q[i % copies][1]), copies * 3)
            row = dict(m=m, n=n, k=k128, tcgen05_us=round(t_mine, 1),
                       tcgen05_gbs=round(n * k128 / (t_mine * 1e-6) / 1e9, 1))
            # activations quantised per token (the reference kernel's numerics): quantise + int8 x int8 product
            t_i8 = graph_time(lambda i: C.w8a16_linear(x, q[i % copies][0], q[i % copies][1], act_int8=True), copies * 3)
            row.update(int8_act_us=round(t_i8, 1), int8_act_gbs=round(n * k128 / (t_i8 * 1e-6) / 1e9, 1))
            # the same with group-128 weight scales (the reference's format)
            qg = [ref.quantize_w8_grouped(t, 128) for t in w]
            t_g = graph_time(lambda i: C.w8a16_linear(x, qg[i % copies][0], qg[i % copies][1], act_int8=True,
                                                      group_scale=qg[i % copies][1]), copies * 3)
            row.update(int8_act_group128_us=round(t_g, 1), int8_act_group128_gbs=round(n * k128 / (t_g * 1e-6) / 1e9, 1))
            if R is not None and m <= 16:
                prep = []
                for wq, s in q:
                    wq_t = wq.view(n, k128 // 16, 16).permute(1, 0, 2).contiguous()
                    sw_t = s.float()[None, :].expand(k128 // 128, n).contiguous()
                    prep.append((wq_t, sw_t))

                def ref_call(i):
                    xq, xs = R.w8a16_quant_act(x)
                    return R.w8a16_gemm(xq, xs, prep[i % copies][0], prep[i % copies][1], n, k128, 1)

                t_ref = graph_time(ref_call, copies * 3)
                row.update(reference_us=round(t_ref, 1), reference_gbs=round(n * k128 / (t_ref * 1e-6) / 1e9, 1),
                           speedup=round(t_ref / t_mine, 2), speedup_int8_act=round(t_ref / t_i8, 2))
            rows.append(row)
            print(row, flush=True)
            del w, q
    out = os.environ.get("BL_BENCH_OUT", "w8a16_bench.json")
    json.dump(rows, open(out, "w"))


if __name__ == "__main__":
    main()
