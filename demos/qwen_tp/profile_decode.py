# SPDX-License-Identifier: MIT
"""Per-op device time of one eager decode step (the op tracer of
barlink_sm86_b200.utils): which kernels a token costs and how many.
Counterpart of demos/qwen_tp/qwen38_int8/profile_decode.py:24-44, which counts
kernels per token with torch.profiler.

    python demos/qwen_tp/profile_decode.py [--model qwen25_7b] [--batch 64] [--ctx 1024] [--quant none]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from barlink_sm86_b200.models import DecodeEngine, Qwen2Config, Qwen2Model  # noqa: E402
from barlink_sm86_b200.parallel import TPComm  # noqa: E402
from barlink_sm86_b200.utils import OpTrace  # noqa: E402

ap = argparse.ArgumentParser()
ap.add_argument("--model", default="qwen25_7b", choices=["qwen25_7b", "tiny"])
ap.add_argument("--quant", default="none", choices=["none", "w8a16", "w4a16"])
ap.add_argument("--batch", type=int, default=64)
ap.add_argument("--ctx", type=int, default=1024)
ap.add_argument("--steps", type=int, default=3)
ap.add_argument("--shard-of", type=int, default=0, help="profile rank 0's shard of this TP degree (no communication)")
a = ap.parse_args()
cuda = torch.cuda.is_available()
dev, dt = ("cuda:0", torch.bfloat16) if cuda else ("cpu", torch.float32)
cfg = Qwen2Config.qwen25_7b() if a.model == "qwen25_7b" else Qwen2Config.tiny()
m = Qwen2Model(cfg, TPComm.single(), dev, dt, seed=0, quant=a.quant,
               shard_of=(a.shard_of, 0) if a.shard_of > 1 else None)
e = DecodeEngine(m, a.batch, a.ctx + a.steps + 8, use_graph=False)
e.set_context(a.ctx)  # the cache content does not matter for timing
for _ in range(2):
    e.step()
with OpTrace() as t:
    for _ in range(a.steps):
        e.step()
print(t.table())
print("kernels per step: %d" % e.launches_per_step)
