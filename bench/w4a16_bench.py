# SPDX-License-Identifier: MIT
"""Int4 weight-only GEMV (GPTQ-v1 tensors) on the MLP shapes of the reference's
int4 demo (demos/qwen_tp/int4linear.py:150-172): device time with CUDA events,
L2 flushed between launches, effective bandwidth over the packed bytes, and
the bf16 tcgen05 linear on the widened weight for comparison.

    python bench/w4a16_bench.py [--rows 1]
"""
import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from barlink_sm86_b200 import ops  # noqa: E402
from barlink_sm86_b200.utils import cuda_time_us  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--rows", type=int, default=1)
a = ap.parse_args()
dev = torch.device("cuda:0")
for k, n in ((5120, 17408), (17408, 5120), (5120, 10240), (5120, 6144), (3584, 37888), (18944, 3584)):
    w = torch.randn(n, k, device=dev) * 0.02
    qw, sc, qz = ops.ref.pack_int4(w)
    x = torch.randn(a.rows, k, device=dev).bfloat16()
    wb = w.bfloat16()
    us4 = cuda_time_us(lambda: ops.w4a16_linear(x, qw, sc, qz))
    us16 = cuda_time_us(lambda: ops.linear(x, wb))
    nbytes = qw.numel() * 4 + sc.numel() * 2 + qz.numel() * 4
    print(json.dumps({"k": k, "n": n, "rows": a.rows, "w4a16_us": round(us4, 2), "w4_gbs": round(nbytes / us4 / 1e3, 1),
                      "bf16_linear_us": round(us16, 2), "speedup_vs_bf16": round(us16 / us4, 2)}))
