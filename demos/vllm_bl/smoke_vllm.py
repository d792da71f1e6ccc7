# SPDX-License-Identifier: MIT
"""vLLM tensor-parallel smoke test over the barlink hook (offline LLM API,
small Qwen2 shape; CUDA-graph capture on unless ENFORCE_EAGER=1).  Counterpart
of the reference's demos/vllm_bl/smoke_vllm.py.  Greedy output with the hook
must equal greedy output with BL_SHIM_OFF=1 (NCCL) for the same dummy weights."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
import common  # noqa: E402


def main():
    backend = common.load_hook()
    from vllm import LLM, SamplingParams

    kw, real = common.model_kwargs("qwen2-1.5b", 512)
    llm = LLM(tensor_parallel_size=int(os.environ.get("TP", "2")),
              enforce_eager=os.environ.get("ENFORCE_EAGER") == "1", gpu_memory_utilization=0.42,
              max_model_len=512, **kw)
    prompt = {"prompt_token_ids": list(range(2000, 2016))}
    out = llm.generate([prompt], SamplingParams(max_tokens=32, temperature=0, ignore_eos=True, detokenize=real))
    print("SMOKE OUTPUT (%s): %r" % (backend, list(out[0].outputs[0].token_ids)), flush=True)


if __name__ == "__main__":  # vLLM spawns its workers: the main module is imported again in each
    main()
