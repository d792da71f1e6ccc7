# SPDX-License-Identifier: MIT
"""Offline vLLM tensor-parallel throughput benchmark over the barlink hook
(BL_SHIM_OFF=1: the same run over NCCL).  Counterpart of the reference's
demos/vllm_bl/bench_27b.py:55-133: LLM.generate on fixed prompts or a
synthetic N-token prompt, tokens/s over the wall clock, decode tokens/s from a
warm re-run, optional speculative (MTP) decoding, fp8 KV cache and chunked
prefill; one JSON artifact per run.

    python demos/vllm_bl/bench_tp.py --tp 2 --prompt-tokens 512 --max-tokens 128
    BL_SHIM_OFF=1 python demos/vllm_bl/bench_tp.py --tp 2 ...          # NCCL baseline
    BENCH_MODEL=/path/to/checkpoint python demos/vllm_bl/bench_tp.py ...
"""
import argparse
import json
import os
import sys
import time

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import common  # noqa: E402


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tp", type=int, default=2)
    ap.add_argument("--shape", default="qwen2.5-7b", choices=sorted(common.SHAPES))
    ap.add_argument("--prompt-tokens", type=int, default=512)
    ap.add_argument("--num-prompts", type=int, default=4)
    ap.add_argument("--max-tokens", type=int, default=128)
    ap.add_argument("--max-model-len", type=int, default=4096)
    ap.add_argument("--max-num-seqs", type=int, default=64)
    ap.add_argument("--gpu-mem", type=float, default=0.85)
    ap.add_argument("--mtp", type=int, default=0, help="speculative tokens (needs a checkpoint with an MTP head)")
    ap.add_argument("--kv-dtype", default=None, help="e.g. fp8_e4m3")
    ap.add_argument("--chunked-prefill", action="store_true")
    ap.add_argument("--warm-repeat", type=int, default=1)
    ap.add_argument("--quantization", default=None,
                    help="a vLLM quantization method; barlink_w8a16 = this library's W8A16 linears")
    ap.add_argument("--out-json", default=None)
    a = ap.parse_args()

    if a.quantization == "barlink_w8a16":
        common.enable_w8a16()
    backend = common.load_hook()
    from vllm import LLM, SamplingParams

    kw, real = common.model_kwargs(a.shape, a.max_model_len)
    kw.update(tensor_parallel_size=a.tp, enforce_eager=os.environ.get("ENFORCE_EAGER") == "1",
              gpu_memory_utilization=a.gpu_mem, max_model_len=a.max_model_len, max_num_seqs=a.max_num_seqs)
    if a.mtp > 0:
        kw["speculative_config"] = {"method": "mtp", "num_speculative_tokens": a.mtp}
    if a.kv_dtype:
        kw["kv_cache_dtype"] = a.kv_dtype
    if a.chunked_prefill:
        kw["enable_chunked_prefill"] = True
    if a.quantization:
        kw["quantization"] = a.quantization
    llm = LLM(**kw)

    import random
    rnd = random.Random(0)
    vocab = common.SHAPES[a.shape]["vocab_size"]
    prompts = [{"prompt_token_ids": [rnd.randrange(1000, vocab - 1000) for _ in range(a.prompt_tokens)]}
               for _ in range(a.num_prompts)]
    sp = SamplingParams(temperature=0, max_tokens=a.max_tokens, ignore_eos=True,
                        detokenize=real)
    t0 = time.perf_counter()
    outs = llm.generate(prompts, sp)
    wall = time.perf_counter() - t0
    gen = sum(len(o.outputs[0].token_ids) for o in outs)
    warm = None
    for _ in range(a.warm_repeat):  # prefix cache makes the re-run decode dominated
        t1 = time.perf_counter()
        llm.generate(prompts, sp)
        w = time.perf_counter() - t1
        warm = w if warm is None else min(warm, w)
    res = {"backend": backend, "tp": a.tp, "model": os.environ.get("BENCH_MODEL") or (a.shape + " (dummy weights)"),
           "prompt_tokens": a.prompt_tokens, "prompts": a.num_prompts, "gen_tokens": gen, "wall_s": wall,
           "tps": gen / wall, "warm_wall_s": warm, "decode_tps": (gen / warm) if warm else None,
           "prefill_s": (wall - warm) if warm else None, "mtp": a.mtp, "kv_dtype": a.kv_dtype, "quantization": a.quantization,
           "enforce_eager": os.environ.get("ENFORCE_EAGER") == "1",
           "first_tokens": list(outs[0].outputs[0].token_ids[:8])}
    print("BENCH RESULT " + json.dumps(res), flush=True)
    out = a.out_json or os.path.join(os.path.dirname(os.path.abspath(__file__)), "bench_tp%d_%s.json" % (a.tp, backend))
    with open(out, "w") as f:
        json.dump(res, f, indent=2)


if __name__ == "__main__":
    main()
