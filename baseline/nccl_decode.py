#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""NCCL + cuBLAS baseline for the headline benchmark.

A restatement, in plain PyTorch library calls, of what the reference's decode
harness does on its NCCL branch (demos/qwen_tp/qwen38_int8/worker.py there:
row-parallel linears finished by `dist.all_reduce` hooks :167-183, vocab-
parallel lm_head with an all_gather :208-241, static KV cache and a CUDA-
graphed step :539-614), for the Qwen2.5-7B shape that bench.py measures:
F.linear (cuBLAS), F.scaled_dot_product_attention, torch elementwise ops,
torch.distributed with the "nccl" backend.  None of this repository's kernels
run here.  Same flags and the same JSON line as bench.py
(`"impl": "nccl_cublas_baseline"`).

    python baseline/nccl_decode.py --gpus 1 --steps 64 --warmup 8
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 \
        baseline/nccl_decode.py --gpus 8 --steps 64 --warmup 8
"""
import argparse
import json
import math
import os
import sys
import time

import torch
import torch.distributed as dist
import torch.nn.functional as F

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

from barlink_sm86_b200.models.qwen2 import Qwen2Config, _randn  # noqa: E402  (config + seeded init only)
from barlink_sm86_b200.parallel.plan import gather_head_cols, gather_heads, head_plan, shard_cols, shard_rows  # noqa: E402


def rope(x, cos, sin):
    h = x.shape[-1] // 2
    x1, x2 = x[..., :h], x[..., h:]
    return torch.cat([x1 * cos - x2 * sin, x2 * cos + x1 * sin], -1)


class Layer:
    def __init__(self, cfg, tp, rank, dev, seed, l):
        H, hd = cfg.hidden, cfg.head_dim
        p = head_plan(cfg.n_heads, cfg.n_kv_heads, tp, rank)
        s = seed * 1000003 + l * 64
        dt = torch.bfloat16
        wq, wk, wv = (_randn((n * hd, H), s + i, dev, dt) for i, n in ((1, cfg.n_heads), (2, cfg.n_kv_heads), (3, cfg.n_kv_heads)))
        self.wqkv = torch.cat([gather_heads(wq, p.q_heads, hd), gather_heads(wk, p.kv_heads, hd),
                               gather_heads(wv, p.kv_heads, hd)], 0).contiguous()
        bq, bk, bv = (_randn((n * hd,), s + i, dev, dt) for i, n in ((4, cfg.n_heads), (5, cfg.n_kv_heads), (6, cfg.n_kv_heads)))
        self.bqkv = torch.cat([gather_heads(bq[:, None], p.q_heads, hd)[:, 0], gather_heads(bk[:, None], p.kv_heads, hd)[:, 0],
                               gather_heads(bv[:, None], p.kv_heads, hd)[:, 0]]).contiguous()
        self.wo = gather_head_cols(_randn((H, cfg.n_heads * hd), s + 7, dev, dt), p.q_heads, hd).contiguous()
        self.wg = shard_rows(_randn((cfg.intermediate, H), s + 8, dev, dt), tp, rank)
        self.wu = shard_rows(_randn((cfg.intermediate, H), s + 9, dev, dt), tp, rank)
        self.wd = shard_cols(_randn((H, cfg.intermediate), s + 10, dev, dt), tp, rank)
        self.ln1 = torch.ones(H, dtype=dt, device=dev)
        self.ln2 = torch.ones(H, dtype=dt, device=dev)
        self.nq, self.nkv = p.nq, p.nkv


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=64)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--prompt", type=int, default=1024)
    ap.add_argument("--reps", type=int, default=5)
    ap.add_argument("--limit", type=int, default=240,
                    help="seconds after which the process dumps its stacks and exits: a stuck collective "
                         "must not hold the GPUs")
    args = ap.parse_args()
    import faulthandler
    faulthandler.dump_traceback_later(args.limit, exit=True)
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    lr = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(lr)
    dev = torch.device("cuda", lr)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", rank=rank, world_size=world)
    cfg = Qwen2Config.qwen25_7b()
    H, hd, B, S = cfg.hidden, cfg.head_dim, args.batch, args.prompt
    layers = [Layer(cfg, world, rank, dev, 0, l) for l in range(cfg.layers)]
    embed = _randn((cfg.vocab, H), 900001, dev, torch.bfloat16)
    head = shard_rows(_randn((cfg.vocab, H), 900002, dev, torch.bfloat16), world, rank)
    ln_f = torch.ones(H, dtype=torch.bfloat16, device=dev)
    nq, nkv = layers[0].nq, layers[0].nkv
    max_len = S + args.steps * 2 + args.warmup * 2 + 16
    g = torch.Generator(device=dev).manual_seed(99)
    kc = [torch.randn(B, nkv, max_len, hd, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in layers]
    vc = [torch.randn(B, nkv, max_len, hd, generator=g, device=dev, dtype=torch.float32).to(torch.bfloat16) for _ in layers]
    ids = torch.randint(0, cfg.vocab, (B,), device=dev)
    pos = torch.full((1,), S, device=dev, dtype=torch.long)
    out_ids = torch.zeros(B, dtype=torch.long, device=dev)
    inv = cfg.theta ** (-torch.arange(0, hd, 2, device=dev, dtype=torch.float32) / hd)
    mask = torch.zeros(1, 1, 1, max_len, dtype=torch.bool, device=dev)
    ar_calls = [0]

    def all_reduce(t):
        if world > 1:
            ar_calls[0] += 1
            dist.all_reduce(t)
        return t

    def step():
        x = F.embedding(ids, embed)
        ang = pos.float()[:, None] * inv[None]
        cos, sin = ang.cos().to(torch.bfloat16), ang.sin().to(torch.bfloat16)
        mask.copy_((torch.arange(max_len, device=dev) <= pos)[None, None, None])
        for L, k_, v_ in zip(layers, kc, vc):
            h = F.rms_norm(x, (H,), L.ln1, cfg.eps)
            qkv = F.linear(h, L.wqkv, L.bqkv).view(B, nq + 2 * nkv, hd)
            q, k, v = qkv[:, :nq], qkv[:, nq:nq + nkv], qkv[:, nq + nkv:]
            q, k = rope(q, cos, sin), rope(k, cos, sin)
            k_.index_copy_(2, pos, k.unsqueeze(2))
            v_.index_copy_(2, pos, v.unsqueeze(2))
            a = F.scaled_dot_product_attention(q.unsqueeze(2), k_, v_, attn_mask=mask, enable_gqa=True)
            x = x + all_reduce(F.linear(a.reshape(B, nq * hd), L.wo))
            h = F.rms_norm(x, (H,), L.ln2, cfg.eps)
            x = x + all_reduce(F.linear(F.silu(F.linear(h, L.wg)) * F.linear(h, L.wu), L.wd))
        h = F.rms_norm(x, (H,), ln_f, cfg.eps)
        logits = F.linear(h, head)
        if world > 1:
            full = torch.empty(world, B, head.shape[0], dtype=logits.dtype, device=dev)
            dist.all_gather_into_tensor(full, logits.contiguous())
            logits = full.permute(1, 0, 2).reshape(B, -1)
        nxt = logits.argmax(-1)
        out_ids.copy_(nxt)
        ids.copy_(nxt % cfg.vocab)
        pos.add_(1)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        for _ in range(3):
            step()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    pos.fill_(S)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        step()
    pos.fill_(S)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    for _ in range(args.warmup):
        graph.replay()
    barrier()
    # same timing procedure as bench.py: sampler first, about a second of untimed stepping, then
    # the K-step region `--reps` times from the same context length, median reported
    from barlink_sm86_b200.utils import ClockSampler
    import statistics
    sampler = ClockSampler(lr)
    sampler.start()
    t_load = time.perf_counter()
    while time.perf_counter() - t_load < 1.0:
        pos.fill_(S)
        for _ in range(8):
            graph.replay()
        torch.cuda.synchronize()
    rep_ms = []
    for _ in range(max(1, args.reps)):
        pos.fill_(S)
        barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            graph.replay()
        e1.record()
        barrier()
        rep_ms.append(e0.elapsed_time(e1))
    clocks = sampler.stop()
    ms = statistics.median(rep_ms)
    pos.fill_(S)
    h_in = torch.zeros(B, dtype=torch.long).pin_memory()
    h_out = torch.zeros(B, dtype=torch.long).pin_memory()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        ids.copy_(h_in, non_blocking=True)
        graph.replay()
        h_out.copy_(out_ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        h_in.copy_(h_out % cfg.vocab)
    barrier()
    e2e = (time.perf_counter() - t0) * 1e3
    t = torch.tensor([ms, e2e], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms, e2e = float(t[0]), float(t[1])
    if rank == 0:
        print(json.dumps({
            "metric": "decode_tokens_per_s", "value": round(B * args.steps / (ms / 1e3), 1), "unit": "tokens/s",
            "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": round(ms / args.steps, 4), "higher_is_better": True, "scaling": "strong",
            "dtype": "bf16", "data": "synthetic", "impl": "nccl_cublas_baseline",
            "config": {"model": cfg.name, "global_batch": B, "seq_len": S, "parallelism": "tp%d" % args.gpus,
                       "kv_cache": "static [B, kv_heads, max_len, head_dim], random-filled", "cuda_graph": True},
            "e2e": {"value": round(B * args.steps / (e2e / 1e3), 1), "unit": "tokens/s",
                    "ms_per_step": round(e2e / args.steps, 4), "h2d_bytes_per_step": B * 8, "d2h_bytes_per_step": B * 8},
            "all_reduce_calls_per_step": ar_calls[0] // max(1, 4),
            "clocks": clocks, "rep_ms_per_step": [round(x / args.steps, 4) for x in rep_ms],
            "nccl_nvls": os.environ.get("NCCL_NVLS_ENABLE", "default (on when the fabric supports it)"),
        }))
    if world > 1:
        # The captured graph holds NCCL kernels of this communicator: release it (and let every
        # replay finish) before the communicator goes away.  Destroying the process group with
        # the graph still alive left the ranks stuck after the result line at 4 GPUs.
        dist.barrier()
        torch.cuda.synchronize()
        graph.reset()
        del graph
        torch.cuda.synchronize()
        dist.barrier()
        sys.stdout.flush()
        faulthandler.cancel_dump_traceback_later()
        faulthandler.dump_traceback_later(30, exit=True)  # a teardown that still sticks ends here
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
