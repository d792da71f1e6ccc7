#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Row-parallel linear + all-reduce at prefill / MMDiT sizes: the GEMM whose epilogue scatters its
output tiles into the owners' staging inboxes plus the kernel that finishes the all-reduce
(`TPComm.row_parallel`), against the same GEMM followed by an all-reduce kernel, against NCCL
(`--backend nccl`: cuBLAS-free too, the GEMM is this library's, only the collective differs).

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 bench/gemm/row_parallel_bench.py

Device-timed inside one CUDA graph of `--iters` calls, maximum over ranks.  The roofline of the
fused pair is the slower of its FLOPs at the measured sustained bf16 rate and the bytes that must
leave each GPU (two-shot: 2 (N-1)/N of the message) at the measured peer-copy rate; the reference
has no counterpart (its row-parallel linears are cuBLAS + an all_reduce hook,
demos/flux2_tp/worker.py:106-123 there).
"""
import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="barlink", choices=["barlink", "nccl"])
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tflops", type=float, default=1357.7, help="sustained bf16 rate used for the roofline")
    ap.add_argument("--link-gbs", type=float, default=770.0, help="peer-copy rate per direction used for the roofline")
    ap.add_argument("--out", default="")
    a = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("BL_POOL_MB", "1024")
    if a.backend == "barlink":
        from barlink_sm86_b200 import process_group as blpg
        blpg.init_process_group(rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world)
    from barlink_sm86_b200.parallel import TPComm
    comm = TPComm(dist.group.WORLD)

    def timed(fn):
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(2):
                fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            for _ in range(a.iters):
                fn()
        g.replay()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        g.replay()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / a.iters], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        del g
        return float(t)

    rows = []
    # (tokens, n, k_full): MMDiT proj / fc2 / single-block out, and the 7B-shape prefill o_proj / down
    for name, T, n, kfull in (("mmdit proj", 4608, 3072, 3072), ("mmdit fc2", 4608, 3072, 12288),
                              ("mmdit single out", 4608, 3072, 12288), ("7b prefill o_proj", 8192, 3584, 3584),
                              ("7b prefill down", 8192, 3584, 18944)):
        k = kfull // world
        k -= k % 8
        gen = torch.Generator(device=dev).manual_seed(rank)
        x = (torch.randn(T, k, device=dev, generator=gen) * 0.5).to(torch.bfloat16)
        w = (torch.randn(n, k, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        out = torch.empty(T, n, dtype=torch.bfloat16, device=dev)
        parts = [(x, w, None, None, False, 0)]
        res = {}
        for mode in (("fused", "1"), ("gemm_then_allreduce", "0")) if a.backend == "barlink" else (("gemm_then_nccl", "0"),):
            os.environ["BL_PUSH_AR"] = mode[1]
            res[mode[0]] = timed(lambda: comm.row_parallel(out, parts))
        os.environ["BL_PUSH_AR"] = "0"
        from barlink_sm86_b200 import ops
        res["gemm_alone"] = timed(lambda: ops.linear(x, w, out=out))
        flops = 2.0 * T * n * k
        nbytes = T * n * 2
        t_flops = flops / (a.tflops * 1e12) * 1e6
        t_link = 2.0 * (world - 1) / world * nbytes / (a.link_gbs * 1e9) * 1e6
        floor = max(t_flops, t_link)
        row = dict(case=name, tokens=T, n=n, k_local=k, world=world, backend=a.backend, us=res,
                   roofline_us=round(floor, 1), flops_us=round(t_flops, 1), link_us=round(t_link, 1))
        if "fused" in res:
            row["fused_fraction_of_roofline"] = round(floor / res["fused"], 3)
        rows.append(row)
        if rank == 0:
            print(json.dumps(row), flush=True)
    if rank == 0 and a.out:
        with open(a.out, "w") as f:
            json.dump(rows, f, indent=1)
    dist.barrier()
    dist.destroy_process_group()
    if a.backend == "barlink":
        import barlink_sm86_b200 as bl
        bl.shutdown()


if __name__ == "__main__":
    main()
