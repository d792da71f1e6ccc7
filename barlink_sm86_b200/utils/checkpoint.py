# SPDX-License-Identifier: MIT
"""Qwen2-style checkpoints in the Hugging Face layout (safetensors shards +
config.json): a tensor source for `Qwen2Weights` that streams each full tensor
from disk when the loader asks for it (so that a rank only ever holds one
unsharded tensor at a time), and an exporter that writes a model of this
library back out under the same names.

The reference streams its checkpoints the same way and shards every tensor
as soon as it is read (demos/qwen_tp/qwen38_int8/worker.py:294-441).

    src = SafetensorsSource("/path/to/Qwen2.5-7B", device, torch.bfloat16)
    model = Qwen2Model(src.config(), comm, device, torch.bfloat16, source=src)
"""
import json
import os

import torch


def config_from_hf(path):
    """Qwen2Config from a Hugging Face config.json (file or directory)."""
    from ..models.qwen2 import Qwen2Config

    if os.path.isdir(path):
        path = os.path.join(path, "config.json")
    with open(path) as f:
        c = json.load(f)
    hidden, heads = c["hidden_size"], c["num_attention_heads"]
    return Qwen2Config(hidden=hidden, layers=c["num_hidden_layers"], n_heads=heads,
                       n_kv_heads=c.get("num_key_value_heads", heads), head_dim=c.get("head_dim", hidden // heads),
                       intermediate=c["intermediate_size"], vocab=c["vocab_size"],
                       eps=c.get("rms_norm_eps", 1e-6), theta=c.get("rope_theta", 1e6),
                       qkv_bias=c.get("attention_bias", c.get("model_type", "qwen2") == "qwen2"),
                       name=c.get("_name_or_path") or c.get("model_type", "qwen2"))


class SafetensorsSource:
    """Full tensors by Hugging Face name from the safetensors shards of a directory."""

    ATTN = ("q_proj", "k_proj", "v_proj", "o_proj")
    MLP = ("gate_proj", "up_proj", "down_proj")

    def __init__(self, directory, device, dtype):
        from safetensors import safe_open

        self.dir, self.device, self.dtype = directory, device, dtype
        self._open = safe_open
        self._handles = {}
        index = os.path.join(directory, "model.safetensors.index.json")
        if os.path.exists(index):
            with open(index) as f:
                self.where = json.load(f)["weight_map"]
        else:
            self.where = {}
            for fn in sorted(os.listdir(directory)):
                if fn.endswith(".safetensors"):
                    with safe_open(os.path.join(directory, fn), framework="pt", device="cpu") as h:
                        for k in h.keys():
                            self.where[k] = fn
        if not self.where:
            raise FileNotFoundError("no safetensors tensors under %s" % directory)
        self.tied = "lm_head.weight" not in self.where

    def config(self):
        return config_from_hf(self.dir)

    def _get(self, key):
        fn = self.where.get(key)
        if fn is None:
            raise KeyError("tensor %r is not in the checkpoint at %s" % (key, self.dir))
        if fn not in self._handles:
            self._handles[fn] = self._open(os.path.join(self.dir, fn), framework="pt", device="cpu")
        return self._handles[fn].get_tensor(key).to(device=self.device, dtype=self.dtype)

    def key(self, name, layer):
        if layer < 0:
            if name == "lm_head.weight":
                return "model.embed_tokens.weight" if self.tied else "lm_head.weight"
            return "model." + name
        part = name.split(".")[0]
        group = "self_attn." if part in self.ATTN else "mlp." if part in self.MLP else ""
        return "model.layers.%d.%s%s" % (layer, group, name)

    def weight(self, name, layer, shape, slot):
        t = self._get(self.key(name, layer))
        if tuple(t.shape) != tuple(shape):
            raise ValueError("%s has shape %s, the configuration expects %s"
                             % (self.key(name, layer), tuple(t.shape), tuple(shape)))
        return t

    def norm(self, name, layer, n):
        return self.weight(name, layer, (n,), 0)


def save_qwen2_safetensors(model, directory, shard_bytes=2 << 30):
    """Write a single-rank (TP=1, unquantised) Qwen2Model as a Hugging Face style checkpoint."""
    from safetensors.torch import save_file

    w, cfg = model.w, model.cfg
    if w.tp != 1 or w.quant != "none":
        raise ValueError("export needs the unsharded bf16/fp32 model (tp=1, quant='none')")
    os.makedirs(directory, exist_ok=True)
    hd, nq, nkv, inter = cfg.head_dim, cfg.n_heads, cfg.n_kv_heads, cfg.intermediate
    tensors = {"model.embed_tokens.weight": w.embed, "lm_head.weight": w.dense(w.lm_head)[: cfg.vocab],
               "model.norm.weight": w.ln_f}
    for l, L in enumerate(w.layers):
        p = "model.layers.%d." % l
        qkv = w.dense(L["wqkv"])
        tensors[p + "self_attn.q_proj.weight"] = qkv[: nq * hd]
        tensors[p + "self_attn.k_proj.weight"] = qkv[nq * hd:(nq + nkv) * hd]
        tensors[p + "self_attn.v_proj.weight"] = qkv[(nq + nkv) * hd:]
        if L["bqkv"] is not None:
            tensors[p + "self_attn.q_proj.bias"] = L["bqkv"][: nq * hd]
            tensors[p + "self_attn.k_proj.bias"] = L["bqkv"][nq * hd:(nq + nkv) * hd]
            tensors[p + "self_attn.v_proj.bias"] = L["bqkv"][(nq + nkv) * hd:]
        tensors[p + "self_attn.o_proj.weight"] = w.dense(L["wo"])
        gu = w.dense(L["wgu"])
        tensors[p + "mlp.gate_proj.weight"] = gu[0::2][:inter]
        tensors[p + "mlp.up_proj.weight"] = gu[1::2][:inter]
        tensors[p + "mlp.down_proj.weight"] = w.dense(L["wdown"])[:, :inter]
        tensors[p + "input_layernorm.weight"] = L["ln1"]
        tensors[p + "post_attention_layernorm.weight"] = L["ln2"]
    shards, cur, size = [], {}, 0
    for k, t in tensors.items():
        t = t.detach().contiguous().cpu()
        n = t.numel() * t.element_size()
        if cur and size + n > shard_bytes:
            shards.append(cur)
            cur, size = {}, 0
        cur[k] = t
        size += n
    shards.append(cur)
    weight_map = {}
    for i, sh in enumerate(shards):
        fn = "model-%05d-of-%05d.safetensors" % (i + 1, len(shards))
        save_file(sh, os.path.join(directory, fn))
        weight_map.update({k: fn for k in sh})
    with open(os.path.join(directory, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {}, "weight_map": weight_map}, f)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump({"architectures": ["Qwen2ForCausalLM"], "model_type": "qwen2", "hidden_size": cfg.hidden,
                   "num_hidden_layers": len(w.layers), "num_attention_heads": nq, "num_key_value_heads": nkv,
                   "head_dim": hd, "intermediate_size": inter, "vocab_size": cfg.vocab, "rms_norm_eps": cfg.eps,
                   "rope_theta": cfg.theta, "attention_bias": cfg.qkv_bias, "tie_word_embeddings": False,
                   "hidden_act": "silu"}, f, indent=2)
    return directory
