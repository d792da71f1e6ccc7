#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Large-message all_reduce bandwidth through the torch.distributed API,
4 MB .. 1 GB (the reference's bench/latency/pg_bw.py:32-47 went to 64 MB)."""
import argparse
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

ap = argparse.ArgumentParser()
ap.add_argument("--backend", default="barlink")
args = ap.parse_args()
rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
os.environ.setdefault("BL_POOL_MB", "4096")
if args.backend == "barlink":
    from barlink_sm86_b200 import process_group as blpg
    blpg.init_process_group(rank=rank, world_size=world)
else:
    dist.init_process_group(args.backend, rank=rank, world_size=world)
for mb in (4, 16, 64, 256, 1024):
    t = torch.zeros(mb << 19, dtype=torch.bfloat16, device="cuda")
    for _ in range(3):
        dist.all_reduce(t)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    n = 10 if mb <= 64 else 4
    e0.record()
    for _ in range(n):
        dist.all_reduce(t)
    e1.record()
    torch.cuda.synchronize()
    ms = torch.tensor([e0.elapsed_time(e1) / n], device="cuda")
    dist.all_reduce(ms, op=dist.ReduceOp.MAX)
    if rank == 0:
        bw = 2 * (world - 1) / world * (mb << 20) / (ms.item() * 1e-3) / 1e9
        print("%s all_reduce %5d MB: %8.3f ms, bus bandwidth %7.1f GB/s" % (args.backend, mb, ms.item(), bw))
dist.barrier()
dist.destroy_process_group()
