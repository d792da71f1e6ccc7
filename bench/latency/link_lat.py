#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Raw link latency, below the process group: `bl.allreduce_into` per algorithm
and the signal round trip, 4 KB .. 4 MB (the reference's bench/latency/
bar_lat.py:19-59 measured copy_ and the pool allreduce_ the same way)."""
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200 import process_group as blpg  # noqa: E402

rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", "0")))
os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
blpg.init_process_group(rank=rank, world_size=world)
info = bl.info()
probe = bl.signal_probe(2000)
if rank == 0:
    print("signal round trip %.2f us, empty launch %.2f us" % (probe[0] / 1e3, probe[1] / 1e3))
for nbytes in (4096, 16384, 65536, 262144, 1 << 20, 4 << 20):
    x = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device="cuda")
    y = torch.empty_like(x)
    line = "%8d B:" % nbytes
    for algo in ("oneshot", "twoshot") + (("nvls",) if info["multicast"] else ()):
        if algo == "oneshot" and nbytes > info["oneshot_max"]:
            continue
        g = torch.cuda.CUDAGraph()
        bl.allreduce_into(y, x, algo)
        torch.cuda.synchronize()
        with torch.cuda.graph(g):
            for _ in range(50):
                bl.allreduce_into(y, x, algo)
        g.replay()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) / 50 * 1e3], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        line += "  %s %.2f us" % (algo, t.item())
    if rank == 0:
        print(line)
dist.barrier()
dist.destroy_process_group()
bl.shutdown()
