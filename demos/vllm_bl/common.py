# SPDX-License-Identifier: MIT
"""Shared pieces of the vLLM demos: loading the barlink hook before vLLM, and
a synthetic model directory for machines without checkpoints.

With `BENCH_MODEL` unset the demos run a Qwen2-shaped model with vLLM's dummy
weights (`load_format="dummy"`) and token-id prompts (`skip_tokenizer_init`),
so the tensor-parallel plumbing -- the part this library replaces -- is
exercised end to end without a checkpoint or a tokenizer."""
import json
import os
import sys
import tempfile

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

SHAPES = {
    "qwen2-1.5b": dict(hidden_size=1536, intermediate_size=8960, num_hidden_layers=28, num_attention_heads=12,
                       num_key_value_heads=2, vocab_size=151936),
    "qwen2.5-32b": dict(hidden_size=5120, intermediate_size=27648, num_hidden_layers=64, num_attention_heads=40,
                        num_key_value_heads=8, vocab_size=152064),
    "qwen2.5-7b": dict(hidden_size=3584, intermediate_size=18944, num_hidden_layers=28, num_attention_heads=28,
                       num_key_value_heads=4, vocab_size=152064),
}


def enable_w8a16():
    """Turn on the hook's quantization step (vLLM quantization="barlink_w8a16": linear layers
    run this library's W8A16 kernel) for this process and the workers it spawns.  Call before load_hook()."""
    steps = os.environ.get("BL_SHIM_STEPS", "1,2,3,4").split(",")
    if "6" not in steps:
        steps.append("6")
    os.environ["BL_SHIM_STEPS"] = ",".join(steps)


def load_hook():
    """Install the barlink hook unless BL_SHIM_OFF=1 (then vLLM keeps NCCL: the A/B baseline)."""
    if ROOT not in sys.path:
        sys.path.insert(0, ROOT)
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    if os.environ.get("BL_SHIM_OFF") != "1":
        # worker processes are spawned: they load the hook through sitecustomize.py on PYTHONPATH
        os.environ["BL_SHIM"] = "1"
        os.environ["PYTHONPATH"] = ROOT + os.pathsep + os.environ.get("PYTHONPATH", "")
        import vllm_barlink  # noqa: F401
        vllm_barlink.install()
    elif "6" in os.environ.get("BL_SHIM_STEPS", "").split(","):
        # the NCCL arm of an A/B run keeps this library's linears: only the quantization method is
        # registered (workers get its classes, and with them the op, when they unpickle the configuration)
        os.environ["PYTHONPATH"] = ROOT + os.pathsep + os.environ.get("PYTHONPATH", "")
        from vllm_barlink import quant
        quant.register()
    return "nccl" if os.environ.get("BL_SHIM_OFF") == "1" else "barlink"


def synthetic_model_dir(shape="qwen2-1.5b", max_len=32768):
    cfg = dict(architectures=["Qwen2ForCausalLM"], model_type="qwen2", hidden_act="silu", rms_norm_eps=1e-6,
               rope_theta=1000000.0, max_position_embeddings=max_len, tie_word_embeddings=False,
               torch_dtype="bfloat16", bos_token_id=151643, eos_token_id=151645, attention_dropout=0.0,
               initializer_range=0.02, use_cache=True, sliding_window=None, use_sliding_window=False)
    cfg.update(SHAPES[shape])
    d = tempfile.mkdtemp(prefix="bl-vllm-%s-" % shape)
    with open(os.path.join(d, "config.json"), "w") as f:
        json.dump(cfg, f, indent=2)
    return d


def model_kwargs(shape="qwen2-1.5b", max_len=32768):
    """LLM(...) keyword arguments that select the model: a real checkpoint from
    BENCH_MODEL, else the synthetic directory with dummy weights."""
    real = os.environ.get("BENCH_MODEL")
    if real:
        return dict(model=real), True
    return dict(model=synthetic_model_dir(shape, max_len), load_format="dummy", skip_tokenizer_init=True), False
