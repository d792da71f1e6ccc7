# SPDX-License-Identifier: MIT
"""Needle-in-a-haystack check at long context through vLLM with tensor
parallelism (fp8 KV cache, chunked prefill): a sentence hidden at
NEEDLE_DEPTH of a NEEDLE_HAYSTACK-word document must be quoted back.
Counterpart of the reference's demos/vllm_bl/needle_check.py:58-66.  Needs a
real checkpoint with a tokenizer (BENCH_MODEL); with dummy weights the answer
would be noise, so without one the script says so and exits 0."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import common  # noqa: E402

DEPTH = float(os.environ.get("NEEDLE_DEPTH", "0.5"))
WORDS = int(os.environ.get("NEEDLE_HAYSTACK", "80000"))
NEEDLE = "The special authorization code for the link project is ZETA-7741-QUANTUM."
QUESTION = ("Based on the document above, what is the special authorization code for the link project? "
            "Reply with just the code.")
FILLER = [
    "System log entry: the transfer between host memory and the device buffer completed within nominal latency.",
    "Maintenance report: cooling loop pressure nominal, fan arrays operating at 42 percent duty cycle.",
    "Meeting notes: the storage migration window is scheduled for next Thursday between 02:00 and 04:00.",
    "Shipping manifest: forty two rack units departed the warehouse with tracking numbers attached.",
    "Field observation: the prototype sensor array recorded stable readings across all twelve channels.",
    "Budget summary: quarterly operational expenses came in 3 percent under the projected envelope.",
    "Lab journal: the calibration run completed after seven iterations with residuals below threshold.",
    "Incident review: the network partition healed automatically once the spanning tree reconverged.",
]


def main():
    model = os.environ.get("BENCH_MODEL")
    if not model:
        print("NEEDLE unavailable: set BENCH_MODEL to a checkpoint directory with a tokenizer")
        return 0
    backend = common.load_hook()
    from transformers import AutoTokenizer
    from vllm import LLM, SamplingParams
    words, i = [], 0
    while len(words) < WORDS:
        words.extend(FILLER[i % len(FILLER)].split())
        i += 1
    words = words[:WORDS]
    pos = int(len(words) * DEPTH)
    doc = " ".join(words[:pos]) + " " + NEEDLE + " " + " ".join(words[pos:])
    tok = AutoTokenizer.from_pretrained(model)
    prompt = tok.apply_chat_template([{"role": "user", "content": doc + "\n\n" + QUESTION}], tokenize=False,
                                     add_generation_prompt=True)
    llm = LLM(model=model, tensor_parallel_size=int(os.environ.get("TP", "2")), gpu_memory_utilization=0.93,
              max_model_len=int(os.environ.get("NEEDLE_MAXLEN", "262144")), max_num_seqs=1,
              kv_cache_dtype="fp8_e4m3", enable_chunked_prefill=True)
    out = llm.generate([prompt], SamplingParams(temperature=0, max_tokens=int(os.environ.get("NEEDLE_MAXTOK", "200"))))
    text = out[0].outputs[0].text
    ok = "ZETA-7741-QUANTUM" in text
    print("NEEDLE RESULT backend=%s depth=%.2f haystack_words=%d ok=%s" % (backend, DEPTH, WORDS, ok), flush=True)
    print("ANSWER: %s" % text.strip()[:200], flush=True)
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
