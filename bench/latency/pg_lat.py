#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""all_reduce latency through the torch.distributed API, 10 KB .. 1 MB, event-
timed and host-sync-timed (the reference's bench/latency/pg_lat.py:36-58:
10 warm-up + 50 timed each way).  --backend barlink|nccl|gloo."""
import argparse
import os
import sys
import time

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

ap = argparse.ArgumentParser()
ap.add_argument("--backend", default="barlink")
ap.add_argument("--sizes", default="10240,65536,262144,1048576")
args = ap.parse_args()
rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
if args.backend == "barlink":
    from barlink_sm86_b200 import process_group as blpg
    blpg.init_process_group(rank=rank, world_size=world)
else:
    dist.init_process_group(args.backend, rank=rank, world_size=world)
for nbytes in [int(s) for s in args.sizes.split(",")]:
    t = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device="cuda")
    for _ in range(10):
        dist.all_reduce(t)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(50):
        dist.all_reduce(t)
    e1.record()
    torch.cuda.synchronize()
    ev = e0.elapsed_time(e1) / 50 * 1e3
    t0 = time.perf_counter()
    for _ in range(50):
        dist.all_reduce(t)
        torch.cuda.synchronize()
    sy = (time.perf_counter() - t0) / 50 * 1e6
    r = torch.tensor([ev, sy], device="cuda")
    dist.all_reduce(r, op=dist.ReduceOp.MAX)
    if rank == 0:
        print("%s all_reduce %8d B: %7.1f us event-timed, %7.1f us sync-timed (max over %d ranks)"
              % (args.backend, nbytes, r[0].item(), r[1].item(), world))
dist.barrier()
dist.destroy_process_group()
