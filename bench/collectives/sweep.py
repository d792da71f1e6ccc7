#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Collective sweep: all-reduce (one-shot, two-shot, NVLS), all-gather and
reduce-scatter from 4 KiB to 1 GiB in bf16 and fp32, plus the fused
all-reduce + residual + RMSNorm at hidden 3584 for 1..256 tokens, on the
barlink link or on NCCL (the reference's A/B arm: bench/latency/nccl_lat.py,
pg_lat.py, pg_bw.py there).  Every number is timed on the device with CUDA
events around `--iters` calls (one captured graph on the link; an eager loop
on NCCL unless --nccl-graph) and reported as the maximum over ranks; bus bandwidth uses the usual 2(N-1)/N factor for all-reduce and
(N-1)/N for the other two.

    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        bench/collectives/sweep.py --backend barlink --out sweep_barlink.json
    ... --backend nccl
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
    ap.add_argument("--min-bytes", type=int, default=4096)
    ap.add_argument("--max-bytes", type=int, default=1 << 30)
    ap.add_argument("--iters", type=int, default=20)
    ap.add_argument("--out", default="")
    ap.add_argument("--dtypes", default="bf16,fp32")
    ap.add_argument("--nccl-graph", action="store_true",
                    help="time NCCL inside a captured graph too (default: eager loop of --iters calls)")
    args = ap.parse_args()
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("BL_POOL_MB", "4096")
    bl = None
    if args.backend == "barlink":
        import barlink_sm86_b200 as bl
        from barlink_sm86_b200 import process_group as blpg
        blpg.init_process_group(rank=rank, world_size=world)
    else:
        dist.init_process_group("nccl", rank=rank, world_size=world)

    def timed(fn, iters):
        """us per call, graph of `iters` calls, max over ranks."""
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(3):
                fn()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        try:
            if args.backend == "nccl" and not args.nccl_graph:
                raise RuntimeError("eager")
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g):
                for _ in range(iters):
                    fn()
            run = g.replay
            n = iters
        except Exception:
            torch.cuda.synchronize()
            run, n = (lambda: [fn() for _ in range(iters)]), iters
        run()
        dist.barrier()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        run()
        e1.record()
        torch.cuda.synchronize()
        t = torch.tensor([e0.elapsed_time(e1) * 1e3 / n], device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t)

    rows = []
    info = bl.info() if bl else {}
    algos = ["auto"]
    if bl:
        algos = ["oneshot", "twoshot"] + (["nvls"] if info.get("multicast") else []) + ["auto"]
    dts = {"bf16": torch.bfloat16, "fp32": torch.float32}
    for dname in args.dtypes.split(","):
        dt = dts[dname]
        size = args.min_bytes
        while size <= args.max_bytes:
            n = size // (2 if dt == torch.bfloat16 else 4)
            x = torch.randn(n, device=dev).to(dt)
            iters = args.iters if size <= (64 << 20) else max(2, args.iters // 5)
            for algo in algos:
                if bl and algo == "oneshot" and size > info["oneshot_max"]:
                    continue
                if bl and size > info["max_chunk"] and algo != "auto":
                    continue
                y = torch.empty_like(x)
                if bl and algo != "auto":
                    fn = lambda: bl.allreduce_into(y, x, algo)  # noqa: E731
                elif bl and size <= info["max_chunk"]:
                    fn = lambda: bl.allreduce_into(y, x)  # noqa: E731
                else:
                    fn = lambda: dist.all_reduce(x)  # noqa: E731
                us = timed(fn, iters)
                rows.append(dict(op="allreduce", algo=algo if bl else "nccl", dtype=dname, bytes=size, us=round(us, 2),
                                 busbw_gbs=round(2 * (world - 1) / world * size / us / 1e3, 2)))
            if size <= (256 << 20):
                per = max(16, size // world // 16 * 16)
                ne = per // x.element_size()
                xin = x[:ne].contiguous()
                out = torch.empty(world * ne, device=dev, dtype=dt)
                us = timed(lambda: dist.all_gather_into_tensor(out, xin), iters)
                rows.append(dict(op="allgather", algo=args.backend, dtype=dname, bytes=per * world, us=round(us, 2),
                                 busbw_gbs=round((world - 1) / world * per * world / us / 1e3, 2)))
                big = torch.randn(world * ne, device=dev).to(dt)
                o2 = torch.empty(ne, device=dev, dtype=dt)
                us = timed(lambda: dist.reduce_scatter_tensor(o2, big), iters)
                rows.append(dict(op="reduce_scatter", algo=args.backend, dtype=dname, bytes=per * world,
                                 us=round(us, 2), busbw_gbs=round((world - 1) / world * per * world / us / 1e3, 2)))
            del x
            size *= 4 if size >= (1 << 20) else 2
    # fused all-reduce + residual + RMSNorm against the unfused sequence
    H = 3584
    gamma = torch.ones(H, device=dev, dtype=torch.bfloat16)
    for tokens in (1, 2, 4, 8, 16, 32, 64, 128, 256):
        x = torch.randn(tokens, H, device=dev).to(torch.bfloat16)
        res = torch.randn(tokens, H, device=dev).to(torch.bfloat16)
        if bl and x.numel() * 2 <= info["oneshot_max"]:
            us = timed(lambda: bl.allreduce_rmsnorm(x, res, gamma, 1e-6), args.iters)
            rows.append(dict(op="allreduce_residual_rmsnorm", algo="fused", dtype="bf16", tokens=tokens,
                             bytes=tokens * H * 2, us=round(us, 2)))

        def unfused():
            y = x.clone()
            dist.all_reduce(y)
            r = y + res
            return torch.nn.functional.rms_norm(r, (H,), gamma, 1e-6)

        us = timed(unfused, args.iters)
        rows.append(dict(op="allreduce_residual_rmsnorm", algo="unfused-" + args.backend, dtype="bf16",
                         tokens=tokens, bytes=tokens * H * 2, us=round(us, 2)))
    if rank == 0:
        print("%-28s %-16s %-5s %12s %10s %10s" % ("op", "algo", "dtype", "bytes", "us", "busbw GB/s"))
        for r in rows:
            print("%-28s %-16s %-5s %12d %10.2f %10s" % (r["op"], r["algo"], r["dtype"], r["bytes"], r["us"],
                                                         r.get("busbw_gbs", "")))
        if args.out:
            with open(args.out, "w") as f:
                json.dump(dict(backend=args.backend, world=world, rows=rows), f)
    dist.barrier()
    dist.destroy_process_group()
    if bl:
        bl.shutdown()


if __name__ == "__main__":
    main()
