#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""send/recv between rank 0 and rank 1 through the torch.distributed API:
ping-pong round trip and full-duplex exchange, 10 KB .. 1 MB (the reference's
bench/latency/pg_p2p_lat.py:29-86)."""
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
if args.backend == "barlink":
    from barlink_sm86_b200 import process_group as blpg
    blpg.init_process_group(rank=rank, world_size=world)
else:
    dist.init_process_group(args.backend, rank=rank, world_size=world)
peer = 1 - rank
for nbytes in (10240, 65536, 262144, 1048576):
    if rank > 1:
        break
    a = torch.zeros(nbytes // 4, device="cuda")
    b = torch.zeros_like(a)
    iters = 100
    for phase in ("pingpong", "duplex"):
        for timed in (False, True):
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            for _ in range(iters if timed else 10):
                if phase == "pingpong":
                    if rank == 0:
                        dist.send(a, peer)
                        dist.recv(b, peer)
                    else:
                        dist.recv(b, peer)
                        dist.send(a, peer)
                else:
                    reqs = [dist.isend(a, peer), dist.irecv(b, peer)]
                    for r in reqs:
                        r.wait()
            e1.record()
            torch.cuda.synchronize()
        if rank == 0:
            us = e0.elapsed_time(e1) / iters * 1e3
            print("%s %-8s %8d B: %7.1f us per %s" % (args.backend, phase, nbytes, us,
                                                      "round trip" if phase == "pingpong" else "exchange"))
dist.barrier()
dist.destroy_process_group()
