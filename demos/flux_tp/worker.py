# SPDX-License-Identifier: MIT
"""Flux-style MMDiT tensor-parallel denoising benchmark, one rank per GPU.

    python demos/flux_tp/worker.py --out results                       # TP=1
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        demos/flux_tp/worker.py --out results                          # TP=2 over the link
    ... worker.py --backend nccl --tag tp2nccl                         # same kernels, NCCL all-reduce

What it measures (same protocol as the reference's worker,
demos/flux2_tp/worker.py:29-42 and :148-160): seeded inputs (image tokens x
channels, text tokens x text dim, timestep 0.5), `--warmup` untimed forwards,
then `--steps` forwards timed one by one with CUDA events; rank 0 saves the
last output and a stats file that compare.py reads.  `--denoise N`
additionally times an N-step sampler run and reports seconds per image.
The model is the library's own MMDiT (random-init weights of the 12B shape:
no checkpoint is read), so every layer runs the sm_100a kernels; the reference
drives the diffusers module with a DTensor plan instead (:106-124).
`--compute-fp32` is the anchor of the reference (:126-132): same bf16 weights,
fp32 arithmetic (the CPU statements of each op, so use it with --config tiny
or be patient).
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def build_inputs(seed, batch, img_tokens, txt_tokens, cfg, dtype):
    from barlink_sm86_b200.models import grid_positions
    g = torch.Generator().manual_seed(seed)
    img = torch.randn(batch, img_tokens, cfg.in_channels, generator=g).to(dtype)
    txt = torch.randn(batch, txt_tokens, cfg.txt_dim, generator=g).to(dtype)
    side = int(round(img_tokens ** 0.5))
    if side * side != img_tokens:
        raise SystemExit("--img-tokens must be a square")
    return img, txt, grid_positions(side, side, "cpu"), torch.full((batch,), 0.5)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--backend", default="barlink", choices=["barlink", "nccl", "gloo"])
    ap.add_argument("--config", default="flux_12b", choices=["flux_12b", "tiny"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--img-tokens", type=int, default=4096)
    ap.add_argument("--txt-tokens", type=int, default=512)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--denoise", type=int, default=0, help="also time a sampler run of this many steps")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--compute-fp32", action="store_true")
    ap.add_argument("--tag", default=None)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()

    import torch.distributed as dist
    from barlink_sm86_b200.models import MMDiTConfig, MMDiTModel, MMDiTWeights, denoise
    from barlink_sm86_b200.parallel import TPComm
    from barlink_sm86_b200 import ops

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    cpu = a.compute_fp32 or a.backend == "gloo"
    dev = torch.device("cpu") if cpu else torch.device("cuda", local)
    if not cpu:
        torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29517")
        if a.backend == "barlink" and not cpu:
            from barlink_sm86_b200 import process_group as blpg
            os.environ.setdefault("BL_POOL_MB", "1024")
            blpg.init_process_group(rank=rank, world_size=world)
        else:
            dist.init_process_group("gloo" if cpu else a.backend, rank=rank, world_size=world)
        comm = TPComm(dist.group.WORLD)
    else:
        comm = TPComm.single()

    cfg = MMDiTConfig.flux_12b() if a.config == "flux_12b" else MMDiTConfig.tiny(hidden=512, heads=4)
    t0 = time.time()
    # weights are always the bf16 values; the anchor only changes the arithmetic
    w = MMDiTWeights(cfg, dev, torch.bfloat16, seed=0, tp=world, rank=rank,
                     gen_device="cpu" if a.config == "tiny" else None)
    model = MMDiTModel(cfg, w, comm)
    load_s = time.time() - t0
    img, txt, pos, t = build_inputs(a.seed, a.batch, a.img_tokens, a.txt_tokens, cfg, torch.bfloat16)
    img, txt, pos, t = img.to(dev), txt.to(dev), pos.to(dev), t.to(dev)

    def sync():
        if not cpu:
            torch.cuda.synchronize()

    def step():
        with torch.inference_mode():
            return model.forward(img, txt, t, pos)

    for _ in range(a.warmup):
        out = step()
    sync()
    times = []
    launches0 = ops.launch_count
    for _ in range(a.steps):
        if cpu:
            t1 = time.perf_counter()
            out = step()
            times.append((time.perf_counter() - t1) * 1e3)
        else:
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            s.record()
            out = step()
            e.record()
            torch.cuda.synchronize()
            times.append(s.elapsed_time(e))
    launches = (ops.launch_count - launches0) // max(1, a.steps)
    if world > 1:  # a step is as slow as its slowest rank
        tt = torch.tensor(times, dtype=torch.float64, device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        times = tt.tolist()
    mean = sum(times) / len(times)

    sec_per_image = None
    if a.denoise > 0:
        sync()
        t1 = time.perf_counter()
        with torch.inference_mode():
            x = denoise(model, img, txt, pos, a.denoise)
        _ = x.float().sum().item()
        sec_per_image = (time.perf_counter() - t1) / a.batch

    tflops = model.flops_per_forward(a.batch, a.img_tokens, a.txt_tokens) / (mean * 1e-3) / 1e12
    mem = 0 if cpu else torch.cuda.max_memory_allocated(dev) / (1 << 30)
    # one write per line: the ranks share the launcher's pipe, and a line written in two pieces gets interleaved
    sys.stdout.write("[tp=%d rank=%d %s] load=%.1fs | %d steps: mean=%.1f ms/step min=%.1f max=%.1f | %.0f TFLOP/s whole job | "
                     "%d kernels/step | peak_mem=%.1f GiB%s\n"
                     % (world, rank, a.backend if world > 1 else "local", load_s, a.steps, mean, min(times), max(times),
                        tflops, launches, mem,
                        "" if sec_per_image is None else " | %d-step sampler: %.2f s/image" % (a.denoise, sec_per_image)))
    sys.stdout.flush()

    tag = a.tag or ("tp%d" % world)
    if rank == 0:
        os.makedirs(a.out, exist_ok=True)
        torch.save(out.float().cpu(), os.path.join(a.out, "output_%s.pt" % tag))
        with open(os.path.join(a.out, "stats_%s.json" % tag), "w") as f:
            json.dump({"tp": world, "backend": a.backend if world > 1 else None, "config": a.config,
                       "compute": "fp32" if a.compute_fp32 else "bf16", "batch": a.batch,
                       "img_tokens": a.img_tokens, "txt_tokens": a.txt_tokens, "steps": a.steps,
                       "warmup": a.warmup, "seed": a.seed, "load_s": load_s, "mean_ms_per_step": mean,
                       "min_ms_per_step": min(times), "max_ms_per_step": max(times), "times_ms": times,
                       "tflops": tflops, "kernels_per_step": launches, "peak_mem_gib": mem,
                       "denoise_steps": a.denoise, "seconds_per_image": sec_per_image,
                       "allreduce_calls_per_step": comm.ar_calls // max(1, a.steps + a.warmup + a.denoise),
                       }, f, indent=2)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
