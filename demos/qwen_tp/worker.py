# SPDX-License-Identifier: MIT
"""Qwen-style tensor-parallel greedy decode benchmark, one rank per GPU.

    python demos/qwen_tp/worker.py --out results                                   # TP=1, bf16
    python -m torch.distributed.run --nproc-per-node 2 --master-addr 127.0.0.1 \
        demos/qwen_tp/worker.py --quant w8a16 --out results                        # TP=2 over the link
    ... worker.py --backend nccl --tag tp2nccl            # same kernels, NCCL collectives
    ... worker.py --no-comm --tag tp2nocomm               # control: collectives skipped

Counterpart of the reference's two decode demos: the INT8 W8A16 worker with
a CUDA-graphed step, `--no-comm` control and step-0 logits dump
(demos/qwen_tp/qwen38_int8/worker.py:462-470, :515-661) and the int4-MLP worker
(demos/qwen_tp/worker.py:409-452).  `--quant w8a16` makes every linear int8
per-channel, `--quant w4a16` makes the MLP int4 (GPTQ-v1, group 128) and the
rest int8.  The model is the library's own decoder with random-init weights of
the named shape (no checkpoint is read), sharded deterministically so that
every TP degree holds the same model.

Rank 0 writes `stats_<tag>.json` (tok/s, ms/token, prefill ms, all-reduce
calls, peak memory), `tokens_<tag>.pt` (generated ids) and `logits_<tag>.pt`
(full-vocabulary logits of the first generated position) for compare.py.
"""
import argparse
import json
import os
import sys
import time

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="qwen25_7b", choices=["qwen25_7b", "qwen25_32b", "tiny"])
    ap.add_argument("--checkpoint", default=None,
                    help="directory with a Hugging Face style Qwen2 checkpoint (safetensors + config.json); "
                         "overrides --model, every rank streams and shards it")
    ap.add_argument("--quant", default="none", choices=["none", "w8a16", "w4a16"])
    ap.add_argument("--backend", default="barlink", choices=["barlink", "nccl", "gloo"])
    ap.add_argument("--batch", type=int, default=1)
    ap.add_argument("--prompt-len", type=int, default=128)
    ap.add_argument("--gen", type=int, default=50, help="timed decode steps")
    ap.add_argument("--warmup", type=int, default=10, help="untimed decode steps")
    ap.add_argument("--no-graph", action="store_true", help="eager step instead of a CUDA graph")
    ap.add_argument("--no-comm", action="store_true", help="control run: skip every collective (wrong results)")
    ap.add_argument("--time-collectives", type=int, default=0, metavar="STEPS",
                    help="after the timed region, run STEPS eager steps on the all-reduce path (one collective "
                         "kernel per row-parallel linear) with CUDA events around every collective and report "
                         "their device time per step")
    ap.add_argument("--layers", type=int, default=0, help="debug: fewer layers")
    ap.add_argument("--seed", type=int, default=1234)
    ap.add_argument("--tag", default=None)
    ap.add_argument("--out", required=True)
    a = ap.parse_args()

    import torch.distributed as dist
    from barlink_sm86_b200 import ops
    from barlink_sm86_b200.models import DecodeEngine, Qwen2Config, Qwen2Model
    from barlink_sm86_b200.parallel import TPComm
    from barlink_sm86_b200.utils import link_stats, max_over_ranks

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    cpu = a.backend == "gloo" or not torch.cuda.is_available()
    dev = torch.device("cpu") if cpu else torch.device("cuda", local)
    if not cpu:
        torch.cuda.set_device(dev)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29541")
        if a.backend == "barlink" and not cpu:
            from barlink_sm86_b200 import process_group as blpg
            os.environ.setdefault("BL_POOL_MB", "1024")
            blpg.init_process_group(rank=rank, world_size=world)
        else:
            dist.init_process_group("gloo" if cpu else a.backend, rank=rank, world_size=world)
        comm = TPComm(dist.group.WORLD)
    else:
        comm = TPComm.single()
    comm.no_comm = a.no_comm

    cfg = {"qwen25_7b": Qwen2Config.qwen25_7b, "qwen25_32b": Qwen2Config.qwen25_32b,
           "tiny": Qwen2Config.tiny}[a.model]()
    dtype = torch.float32 if cpu else torch.bfloat16
    t0 = time.time()
    source = None
    if a.checkpoint:
        from barlink_sm86_b200.utils import SafetensorsSource
        source = SafetensorsSource(a.checkpoint, dev, dtype)
        cfg = source.config()
    model = Qwen2Model(cfg, comm, dev, dtype, seed=0, layers=a.layers or None, quant=a.quant, source=source)
    load_s = time.time() - t0

    g = torch.Generator().manual_seed(a.seed)
    prompts = torch.randint(0, cfg.vocab, (a.batch, a.prompt_len), generator=g, dtype=torch.int32).to(dev)
    total = a.prompt_len + a.warmup + a.gen + 2
    eng = DecodeEngine(model, a.batch, total, use_graph=not a.no_graph)

    def sync():
        if not cpu:
            torch.cuda.synchronize()

    sync()
    t0 = time.perf_counter()
    first = eng.prefill(prompts)
    sync()
    prefill_ms = (time.perf_counter() - t0) * 1e3
    # full-vocabulary logits of the first generated position (what compare.py checks)
    hidden = model.prefill(prompts[:, : a.prompt_len])
    logits0 = model.logits(hidden.view(a.batch, a.prompt_len, -1)[:, -1].contiguous()).float().cpu()

    eng.ids.copy_(first)
    eng.capture()
    toks = [first.clone()]
    for _ in range(a.warmup):
        toks.append(eng.step().clone())
    sync()
    ar0 = comm.ar_calls
    if cpu:
        t0 = time.perf_counter()
        for _ in range(a.gen):
            toks.append(eng.step().clone())
        decode_ms = (time.perf_counter() - t0) * 1e3
    else:
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(a.gen):
            toks.append(eng.step().clone())
        e.record()
        torch.cuda.synchronize()
        decode_ms = s.elapsed_time(e)
    decode_ms = max_over_ranks(decode_ms, device=dev)
    ms_tok = decode_ms / a.gen
    tps = a.batch * 1e3 / ms_tok
    mem = 0.0 if cpu else torch.cuda.max_memory_allocated(dev) / (1 << 30)
    mode = "local" if world == 1 else (a.backend + ("/no-comm" if a.no_comm else ""))
    print("[tp=%d rank=%d %s %s %s] load=%.1fs prefill=%.1f ms | decode %d steps x batch %d: %.3f ms/step, %.1f tok/s | "
          "%d kernels/step (%s) | peak_mem=%.1f GiB"
          % (world, rank, mode, cfg.name, a.quant, load_s, prefill_ms, a.gen, a.batch, ms_tok, tps,
             eng.launches_per_step, "eager" if eng.graph is None else "one graph replay", mem), flush=True)

    # device time of the collectives themselves, call by call (eager, unfused path)
    coll = {"calls_per_step": 0, "device_ms_per_step": 0.0, "steps": 0}
    if a.time_collectives > 0 and world > 1 and not cpu and not a.no_comm:
        saved = os.environ.get("BL_DLIN")
        os.environ["BL_DLIN"] = "0"
        eng2 = DecodeEngine(model, a.batch, total, use_graph=False)
        eng2.cache = eng.cache
        eng2.set_context(a.prompt_len)
        eng2.ids.copy_(first)
        for _ in range(2):
            eng2.step()
        comm.time_collectives = True
        comm.collective_ms()
        for _ in range(a.time_collectives):
            eng2.step()
        n, ms = comm.collective_ms()
        comm.time_collectives = False
        if saved is None:
            os.environ.pop("BL_DLIN", None)
        else:
            os.environ["BL_DLIN"] = saved
        ms = max_over_ranks(ms, device=dev)
        coll = {"calls_per_step": n // a.time_collectives, "device_ms_per_step": ms / a.time_collectives,
                "steps": a.time_collectives}
        if rank == 0:
            print("[tp=%d] collectives on the all-reduce path: %d calls/step, %.3f ms of device time per step "
                  "(eager, max over ranks)" % (world, coll["calls_per_step"], coll["device_ms_per_step"]), flush=True)

    tag = a.tag or ("tp%d%s" % (world, "" if a.quant == "none" else "_" + a.quant))
    if rank == 0:
        os.makedirs(a.out, exist_ok=True)
        torch.save(torch.stack(toks, 1).cpu(), os.path.join(a.out, "tokens_%s.pt" % tag))
        torch.save(logits0, os.path.join(a.out, "logits_%s.pt" % tag))
        with open(os.path.join(a.out, "stats_%s.json" % tag), "w") as f:
            json.dump({"tp": world, "backend": a.backend if world > 1 else None, "no_comm": a.no_comm,
                       "model": cfg.name, "quant": a.quant, "batch": a.batch, "prompt_len": a.prompt_len,
                       "gen": a.gen, "warmup": a.warmup, "graph": eng.graph is not None, "load_s": load_s,
                       "prefill_ms": prefill_ms, "decode_ms_per_token": ms_tok, "tokens_per_s": tps,
                       "kernels_per_step": eng.launches_per_step,
                       "allreduce_calls_timed": comm.ar_calls - ar0, "peak_mem_gib": mem,
                       "decode_path": ("folded" if model.dlin_ok(a.batch) else "fused_rs_ag" if model.fused_ok(a.batch)
                                       else "allreduce"),
                       "collectives_eager": coll,
                       "weight_gib": model.w.nbytes() / (1 << 30), "link": link_stats()}, f, indent=2)
    if world > 1:
        # captured graphs hold references to the communicator's kernels: drop them first
        del eng
        sync()
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
