# SPDX-License-Identifier: MIT
"""Continuous-batching serving benchmark through vLLM's async engine with the
barlink hook (BL_SHIM_OFF=1: the same run over NCCL): N synthetic requests
with prompt lengths uniform in [--prompt-min, --prompt-max], output lengths
uniform in [--out-min, --out-max] and Poisson arrivals at --rate requests/s.
Reports request and token throughput, time to first token and time per output
token (mean and percentiles), and end-to-end latency percentiles.

    python demos/vllm_bl/serve_bench.py --tp 8 --shape qwen2.5-32b --rate 4
    for r in 1 2 4 8 16; do python demos/vllm_bl/serve_bench.py --tp 8 --rate $r; done

Weights are vLLM's dummy weights of the named shape unless BENCH_MODEL points
at a checkpoint; prompts are random token ids (no tokenizer is needed).  The
reference has no serving benchmark (its vLLM numbers come from offline
`LLM.generate`, demos/vllm_bl/bench_27b.py:72-107); this script measures the
same stack under arrival-driven load.
"""
import argparse
import asyncio
import json
import os
import random
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import common  # noqa: E402


def pct(xs, p):
    if not xs:
        return None
    xs = sorted(xs)
    k = min(len(xs) - 1, max(0, int(round(p / 100.0 * (len(xs) - 1)))))
    return xs[k]


async def run(a, backend):
    from vllm import SamplingParams
    from vllm.engine.arg_utils import AsyncEngineArgs
    from vllm.v1.engine.async_llm import AsyncLLM

    kw, real = common.model_kwargs(a.shape, a.max_model_len)
    args = AsyncEngineArgs(tensor_parallel_size=a.tp, max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs,
                           gpu_memory_utilization=a.gpu_mem, enforce_eager=os.environ.get("ENFORCE_EAGER") == "1",
                           enable_chunked_prefill=True, disable_log_stats=True, **kw)
    if a.kv_dtype:
        args.kv_cache_dtype = a.kv_dtype
    if a.quantization:
        args.quantization = a.quantization
    engine = AsyncLLM.from_engine_args(args)
    rnd = random.Random(a.seed)
    vocab = common.SHAPES[a.shape]["vocab_size"]
    reqs, t = [], 0.0
    for i in range(a.requests):
        t += rnd.expovariate(a.rate)
        plen, olen = rnd.randint(a.prompt_min, a.prompt_max), rnd.randint(a.out_min, a.out_max)
        reqs.append((t, [rnd.randrange(1000, vocab - 1000) for _ in range(plen)], olen))
    results = []

    async def one(i, arrival, ids, olen, t0):
        await asyncio.sleep(max(0.0, arrival - (time.perf_counter() - t0)))
        sp = SamplingParams(temperature=0, max_tokens=olen, ignore_eos=True, detokenize=real)
        start = time.perf_counter()
        first, n = None, 0
        async for out in engine.generate({"prompt_token_ids": ids}, sp, request_id="r%d" % i):
            n = len(out.outputs[0].token_ids)
            if first is None and n > 0:
                first = time.perf_counter()
        end = time.perf_counter()
        results.append({"prompt": len(ids), "out": n, "ttft": (first or end) - start, "latency": end - start,
                        "tpot": ((end - first) / (n - 1)) if first and n > 1 else None})

    t0 = time.perf_counter()
    await asyncio.gather(*[one(i, arr, ids, olen, t0) for i, (arr, ids, olen) in enumerate(reqs)])
    wall = time.perf_counter() - t0
    engine.shutdown()
    out_tokens = sum(r["out"] for r in results)
    tpots = [r["tpot"] for r in results if r["tpot"] is not None]
    res = {"backend": backend, "tp": a.tp, "model": os.environ.get("BENCH_MODEL") or (a.shape + " (dummy weights)"),
           "quantization": a.quantization, "requests": len(results), "rate_req_s": a.rate, "wall_s": wall,
           "req_per_s": len(results) / wall, "out_tok_per_s": out_tokens / wall,
           "total_tok_per_s": (out_tokens + sum(r["prompt"] for r in results)) / wall,
           "ttft_ms": {k: 1e3 * pct([r["ttft"] for r in results], p) for k, p in (("p50", 50), ("p90", 90), ("p99", 99))},
           "tpot_ms": {k: 1e3 * pct(tpots, p) for k, p in (("p50", 50), ("p90", 90), ("p99", 99))} if tpots else None,
           "latency_s": {k: pct([r["latency"] for r in results], p) for k, p in (("p50", 50), ("p90", 90), ("p99", 99))}}
    print("SERVE RESULT " + json.dumps(res), flush=True)
    out = a.out_json or os.path.join(os.path.dirname(os.path.abspath(__file__)),
                                     "serve_tp%d_%s_rate%g.json" % (a.tp, backend, a.rate))
    with open(out, "w") as f:
        json.dump(res, f, indent=2)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=8)
    ap.add_argument("--shape", default="qwen2.5-32b", choices=sorted(common.SHAPES))
    ap.add_argument("--requests", type=int, default=512)
    ap.add_argument("--rate", type=float, default=4.0, help="mean arrivals per second (Poisson)")
    ap.add_argument("--prompt-min", type=int, default=128)
    ap.add_argument("--prompt-max", type=int, default=2048)
    ap.add_argument("--out-min", type=int, default=64)
    ap.add_argument("--out-max", type=int, default=512)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=256)
    ap.add_argument("--gpu-mem", type=float, default=0.85)
    ap.add_argument("--kv-dtype", default=None)
    ap.add_argument("--quantization", default=None, help="a vLLM quantization method; barlink_w8a16 = this library's W8A16 linears")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out-json", default=None)
    a = ap.parse_args()
    if a.quantization == "barlink_w8a16":
        common.enable_w8a16()
    backend = common.load_hook()
    asyncio.run(run(a, backend))


if __name__ == "__main__":
    main()
