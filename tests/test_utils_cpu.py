# SPDX-License-Identifier: MIT
"""Observability helpers on CPU: the op tracer restores what it patches, the
clock sampler parses nvidia-smi rows and flags throttle reasons."""
import torch

from barlink_sm86_b200 import ops
from barlink_sm86_b200.utils import ClockSampler, OpTrace, link_stats, max_over_ranks


def test_op_trace_records_and_restores():
    before = ops.linear
    with OpTrace(capacity=4) as t:
        x, w = torch.randn(4, 8), torch.randn(6, 8)
        for _ in range(3):
            ops.linear(x, w)
        ops.rmsnorm(x, torch.ones(8), 1e-6)
        ops.silu_mul(torch.randn(2, 8))
    assert ops.linear is before
    agg = t.summary()
    assert len(t.records) == 4                      # ring buffer keeps the newest records
    assert agg["linear"]["count"] == 2 and agg["rmsnorm"]["count"] == 1 and agg["silu_mul"]["count"] == 1
    assert agg["linear"]["bytes"] == 2 * (4 * 8 + 6 * 8) * 4
    assert "linear" in t.table()


def test_clock_sampler_parse():
    text = ("0, 1905, 1965, 812.33, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
            "0, 1410, 1965, 990.10, 0x0000000000000004, Not Active, Active, Not Active, Active\n"
            "garbage line\n")
    r = ClockSampler.parse(text)
    assert r["samples"] == 2 and r["sm_max_mhz"] == 1965.0 and r["sm_mhz"] == (1905 + 1410) / 2
    assert r["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]


def test_helpers_without_a_link():
    assert isinstance(link_stats(), dict)
    assert max_over_ranks(3.5) == 3.5


def test_safetensors_source_names_and_tied_head(tmp_path):
    """Hugging Face names per tensor, and a checkpoint without lm_head.weight (tied embeddings)
    serves the embedding table as the head."""
    import json

    from safetensors.torch import save_file

    from barlink_sm86_b200.utils import SafetensorsSource, config_from_hf
    d = str(tmp_path)
    emb = torch.randn(32, 16)
    save_file({"model.embed_tokens.weight": emb, "model.norm.weight": torch.ones(16),
               "model.layers.0.self_attn.q_proj.weight": torch.randn(16, 16),
               "model.layers.0.mlp.down_proj.weight": torch.randn(16, 24),
               "model.layers.0.input_layernorm.weight": torch.ones(16)}, d + "/model.safetensors")
    json.dump({"model_type": "qwen2", "hidden_size": 16, "num_hidden_layers": 1, "num_attention_heads": 2,
               "num_key_value_heads": 1, "intermediate_size": 24, "vocab_size": 32, "rope_theta": 10000.0,
               "rms_norm_eps": 1e-5}, open(d + "/config.json", "w"))
    cfg = config_from_hf(d)
    assert (cfg.hidden, cfg.layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.intermediate, cfg.vocab) == \
        (16, 1, 2, 1, 8, 24, 32) and cfg.qkv_bias and cfg.theta == 10000.0 and cfg.eps == 1e-5
    src = SafetensorsSource(d, "cpu", torch.float32)
    assert src.tied
    assert src.key("q_proj.weight", 0) == "model.layers.0.self_attn.q_proj.weight"
    assert src.key("down_proj.weight", 3) == "model.layers.3.mlp.down_proj.weight"
    assert src.key("input_layernorm.weight", 0) == "model.layers.0.input_layernorm.weight"
    assert src.key("norm.weight", -1) == "model.norm.weight"
    assert torch.equal(src.weight("lm_head.weight", -1, (32, 16), 0), emb)
    assert torch.equal(src.norm("norm.weight", -1, 16), torch.ones(16))
    try:
        src.weight("q_proj.weight", 0, (8, 16), 1)
        raise AssertionError("a shape mismatch must be reported")
    except ValueError:
        pass
