# SPDX-License-Identifier: MIT
"""Long-context retrieval check through vLLM with tensor parallelism.

A generated inventory ledger (seeded, procedurally built from word lists, so
no two lines repeat verbatim) hides one or more records whose value is a
random token drawn at run time; the model is asked for the value that belongs
to a given record key and must quote it.  Several depths are probed in one
engine start and the outcome is a JSON line plus an exit code.

The reference has a script of the same purpose (demos/vllm_bl/needle_check.py
there: one fixed sentence in a repeated filler text at 262 144 tokens of
context, fp8 KV cache, chunked prefill).  This one keeps the idea (retrieval at
a chosen depth of a long prompt, served with TP over the hook or, with
BL_SHIM_OFF=1, over NCCL) and nothing of its text or flow.

Needs a real checkpoint with a tokenizer (BENCH_MODEL); dummy weights answer
with noise, so without one the script reports that and exits 0.

Environment: NEEDLE_TOKENS (approximate prompt length, default 200000),
NEEDLE_DEPTHS (comma list of 0..1 fractions, default 0.1,0.5,0.9),
NEEDLE_SEED, NEEDLE_MAXLEN (engine context), TP.
"""
import json
import os
import random
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import common  # noqa: E402

SITES = ("north depot", "harbour annex", "ridge store", "canal yard", "mill loft", "quarry shed", "orchard barn")
ITEMS = ("copper elbows", "ceramic fuses", "hemp rope", "brass valves", "oak dowels", "glass lenses", "felt pads",
         "steel rivets", "linen filters", "rubber gaskets", "tin funnels", "cedar shims")
VERBS = ("counted", "moved", "re-shelved", "weighed", "re-labelled", "inspected", "set aside", "boxed")
NOTES = ("no damage seen", "two crates damp", "label faded", "seal intact", "pallet leaning", "awaiting sign-off",
         "matches last audit", "short by a handful")


def ledger_line(rng, n):
    """One filler record; the running number keeps every line distinct."""
    return "Entry %06d: %d %s %s at the %s, %s." % (
        n, rng.randint(2, 980), rng.choice(ITEMS), rng.choice(VERBS), rng.choice(SITES), rng.choice(NOTES))


def make_secret(rng):
    """(key, value): the record to find and the token that must be quoted back."""
    key = "locker %s-%03d" % (rng.choice("ABCDEFGHJK"), rng.randint(0, 999))
    alphabet = "bcdfghjkmnpqrstvwxz2456789"
    value = "".join(rng.choice(alphabet) for _ in range(4)) + "-" + "".join(rng.choice(alphabet) for _ in range(5))
    return key, value


def build_prompts(tok, target_tokens, depths, seed):
    """One (prompt, key, value, depth) per depth; the ledger is grown line by line until the
    tokenizer says the budget is met, measured on a sample so that tokenisation stays cheap."""
    rng = random.Random(seed)
    sample = [ledger_line(rng, i) for i in range(200)]
    per_line = max(1.0, len(tok("\n".join(sample))["input_ids"]) / 200.0)
    n_lines = max(10, int(target_tokens / per_line))
    cases = []
    for d in depths:
        r = random.Random(seed * 7919 + int(d * 1000))
        lines = [ledger_line(r, i) for i in range(n_lines)]
        key, value = make_secret(r)
        at = min(n_lines - 1, max(0, int(round(d * n_lines))))
        lines.insert(at, "Entry %06d: the combination kept for %s reads %s." % (at, key, value))
        ask = ("The ledger above mentions a combination kept for %s. Answer with that combination only, "
               "exactly as written." % key)
        body = "\n".join(lines) + "\n\n" + ask
        prompt = tok.apply_chat_template([{"role": "user", "content": body}], tokenize=False,
                                         add_generation_prompt=True)
        cases.append((prompt, key, value, d))
    return cases


def main():
    model = os.environ.get("BENCH_MODEL")
    if not model:
        print(json.dumps({"needle": "unavailable", "why": "set BENCH_MODEL to a checkpoint directory with a tokenizer"}))
        return 0
    backend = common.load_hook()
    from transformers import AutoTokenizer
    from vllm import LLM, SamplingParams

    depths = [float(x) for x in os.environ.get("NEEDLE_DEPTHS", "0.1,0.5,0.9").split(",") if x.strip()]
    target = int(os.environ.get("NEEDLE_TOKENS", "200000"))
    seed = int(os.environ.get("NEEDLE_SEED", "17"))
    tok = AutoTokenizer.from_pretrained(model)
    cases = build_prompts(tok, target, depths, seed)
    engine = LLM(model=model, tensor_parallel_size=int(os.environ.get("TP", "2")),
                 max_model_len=int(os.environ.get("NEEDLE_MAXLEN", str(target + 8192))),
                 max_num_seqs=len(cases), kv_cache_dtype=os.environ.get("NEEDLE_KV_DTYPE", "fp8"),
                 enable_chunked_prefill=True, gpu_memory_utilization=float(os.environ.get("NEEDLE_MEM", "0.9")))
    outs = engine.generate([c[0] for c in cases], SamplingParams(temperature=0.0, max_tokens=48))
    rows, all_ok = [], True
    for (prompt, key, value, depth), o in zip(cases, outs):
        text = o.outputs[0].text.strip()
        hit = value in text
        all_ok = all_ok and hit
        rows.append({"depth": depth, "key": key, "expected": value, "answer": text[:80], "found": hit,
                     "prompt_tokens": len(o.prompt_token_ids)})
    print(json.dumps({"needle": "ok" if all_ok else "missed", "backend": backend, "cases": rows}), flush=True)
    return 0 if all_ok else 1


if __name__ == "__main__":
    sys.exit(main())
