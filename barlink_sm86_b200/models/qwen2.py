# SPDX-License-Identifier: MIT
"""Qwen2-style decoder with tensor parallelism, paged KV cache and a
CUDA-graphed decode step.

The reference runs HF `transformers` Qwen models and patches them from the
outside: linears are swapped for quantised ones and row-parallel modules get
an all-reduce hook (demos/qwen_tp/qwen38_int8/worker.py:248-441), the
lm_head is vocab-parallel with an exchange (:208-241), decode is captured in a
CUDA graph with a static cache (:539-614).  There is no network on the build
machines and no checkpoints, so this model owns its layers instead: weights
are random-init N(0, 0.02) from a seed, generated as FULL tensors and then
sharded, so TP=N and TP=1 hold the same model.

Per layer and decode step (CUDA): fused add+RMSNorm (TP: fused with the
all-reduce over NVLink), QKV GEMM with bias, RoPE + paged KV write, paged
attention, o_proj GEMM, fused add+RMSNorm, gate/up GEMM with SiLU*mul in the
epilogue, down GEMM.  All GEMMs are tcgen05 kernels.
"""
import math
from dataclasses import dataclass, field
from typing import Optional

import torch

from .. import ops
from ..parallel import TPComm, head_plan, interleave_gate_up, shard_cols, shard_rows
from ..parallel.plan import gather_head_cols, gather_heads


# BL_DLIN when the environment does not set it: "auto" = the folded-collective decode path whenever
# there is more than one rank, "0" = the k-split GEMM + all-reduce kernel path, "tuned" = the folded
# path at the tensor-parallel degrees listed in DLIN_TUNED_WORLDS.  Measured on B200s (7B shape,
# batch 64, ms per step, folded / k-split): 4.93 / 4.30 on one GPU, 3.31 / 3.44 on two, 2.72 / 2.56 on
# four, 2.65 / 2.36 on eight: the folded path pays at two ranks only.
DLIN_DEFAULT = "tuned"
DLIN_TUNED_WORLDS = (2,)


@dataclass
class Qwen2Config:
    hidden: int = 3584
    layers: int = 28
    n_heads: int = 28
    n_kv_heads: int = 4
    head_dim: int = 128
    intermediate: int = 18944
    vocab: int = 152064
    eps: float = 1e-6
    theta: float = 1e6
    qkv_bias: bool = True
    name: str = "qwen2.5-7b-shape"

    @staticmethod
    def qwen25_7b():
        return Qwen2Config()

    @staticmethod
    def qwen25_32b():
        return Qwen2Config(hidden=5120, layers=64, n_heads=40, n_kv_heads=8, head_dim=128,
                           intermediate=27648, vocab=152064, name="qwen2.5-32b-shape")

    @staticmethod
    def tiny():
        # the plumbing config: hidden 512, 4 layers, 8 query / 2 KV heads, head_dim 64
        return Qwen2Config(hidden=512, layers=4, n_heads=8, n_kv_heads=2, head_dim=64,
                           intermediate=1376, vocab=32000, name="tiny-qwen2")


class W8Weight:
    """int8 weight [n, k] with one bf16 scale per output channel (W8A16)."""
    __slots__ = ("wq", "scale", "shape")

    def __init__(self, w, scale=None):
        """scale: per-row scales to use (a row-parallel shard passes the scales
        of the unsharded rows, so that every shard quantises to the same values
        as the whole weight); None = from the rows of w."""
        if scale is None:
            self.wq, self.scale = ops.ref.quantize_w8(w)
        else:
            self.scale = scale
            self.wq = torch.round(w.float() / scale.float()[:, None]).clamp(-127, 127).to(torch.int8)
        self.shape = tuple(w.shape)

    def numel(self):
        return self.wq.numel() // 2 + self.scale.numel()  # in bf16-element units of memory

    def dense(self):
        return (self.wq.float() * self.scale.float()[:, None]).to(self.scale.dtype)


class W4Weight:
    """GPTQ-v1 int4 weight (group 128): the reference's Int4Linear format
    (demos/qwen_tp/int4linear.py:5-12)."""
    __slots__ = ("qw", "sc", "qz", "group", "shape")

    def __init__(self, w, group=128):
        self.qw, self.sc, self.qz = ops.ref.pack_int4(w, group)
        self.group, self.shape = group, tuple(w.shape)

    def numel(self):
        return self.qw.numel() * 2 + self.sc.numel() + self.qz.numel() * 2

    def dense(self):
        return ops.ref.w4_dequant(self.qw, self.sc, self.qz, self.group).to(torch.bfloat16)


def qlinear(x, w, bias=None, silu_mul=False, split=False):
    """x @ w.T for any stored form of w (plain / tiled bf16, W8Weight, W4Weight).
    split=True allows the k-split slab output of the bf16 decode GEMM."""
    if isinstance(w, W8Weight):
        return ops.w8a16_linear(x, w.wq, w.scale, bias, silu_mul)
    if isinstance(w, W4Weight):
        y = ops.w4a16_linear(x, w.qw, w.sc, w.qz, w.group)
        if bias is not None:
            y = y + bias
        return ops.silu_mul(y, interleaved=True) if silu_mul else y
    if split and bias is None and not silu_mul:
        return ops.linear_split(x, w)
    return ops.linear(x, w, bias, silu_mul=silu_mul)


def _randn(shape, seed, device, dtype, std=0.02):
    g = torch.Generator(device=device)
    g.manual_seed(seed)
    return (torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std).to(dtype)


class RandomSource:
    """Full (unsharded) tensors of a seeded random-init model: N(0, 0.02) weights and biases,
    unit norm weights.  Every tensor has its own generator seed, so any rank can draw any
    tensor without drawing the others."""

    def __init__(self, seed, device, dtype):
        self.base, self.device, self.dtype = seed * 1000003, device, dtype

    def weight(self, name, layer, shape, slot):
        off = self.base + layer * 64 + slot if layer >= 0 else self.base + slot
        return _randn(shape, off, self.device, self.dtype)

    def norm(self, name, layer, n):
        return torch.ones(n, dtype=self.dtype, device=self.device)


class Qwen2Weights:
    """Per-rank shards of a model: seeded random-init by default, or the tensors of `source`
    (an object with `weight(name, layer, shape, slot)` and `norm(name, layer, n)` that returns
    FULL tensors, e.g. `utils.checkpoint.SafetensorsSource`)."""

    def __init__(self, cfg: Qwen2Config, tp: int, rank: int, device, dtype, seed: int = 0,
                 layers: Optional[int] = None, tiled: Optional[bool] = None, quant: str = "none", source=None):
        """quant: "none" (bf16), "w8a16" (every linear int8 per-channel, the
        reference's INT8 demo, demos/qwen_tp/qwen38_int8/worker.py:97-150) or
        "w4a16" (MLP int4 group-128, the rest int8: demos/qwen_tp/worker.py:1-25).
        Quantisation is per output row / per (row, group), so a shard quantises
        to the same values as the matching rows of the unsharded weight."""
        self.cfg, self.tp, self.rank = cfg, tp, rank
        if quant not in ("none", "w8a16", "w4a16"):
            raise ValueError("quant must be none, w8a16 or w4a16")
        self.quant = quant
        if tiled is None:
            import os
            tiled = (torch.device(device).type == "cuda" and dtype == torch.bfloat16
                     and os.environ.get("BL_TILED_WEIGHTS", "0") == "1")
        self.tiled = tiled
        H, hd = cfg.hidden, cfg.head_dim
        self.plan = head_plan(cfg.n_heads, cfg.n_kv_heads, tp, rank)
        n_layers = cfg.layers if layers is None else layers
        self.layers = []
        src = source if source is not None else RandomSource(seed, device, dtype)
        unit = tp * (128 if quant == "w4a16" else 8)  # shards stay 16-byte multiples (int4: whole groups)
        inter_pad = -(-cfg.intermediate // unit) * unit
        self.inter_local = inter_pad // tp
        for l in range(n_layers):
            wq = src.weight("q_proj.weight", l, (cfg.n_heads * hd, H), 1)
            wk = src.weight("k_proj.weight", l, (cfg.n_kv_heads * hd, H), 2)
            wv = src.weight("v_proj.weight", l, (cfg.n_kv_heads * hd, H), 3)
            wqkv = torch.cat([gather_heads(wq, self.plan.q_heads, hd),
                              gather_heads(wk, self.plan.kv_heads, hd),
                              gather_heads(wv, self.plan.kv_heads, hd)], 0).contiguous()
            del wq, wk, wv
            bqkv = None
            if cfg.qkv_bias:
                bq = src.weight("q_proj.bias", l, (cfg.n_heads * hd,), 4)
                bk = src.weight("k_proj.bias", l, (cfg.n_kv_heads * hd,), 5)
                bv = src.weight("v_proj.bias", l, (cfg.n_kv_heads * hd,), 6)
                bqkv = torch.cat([gather_heads(bq[:, None], self.plan.q_heads, hd)[:, 0],
                                  gather_heads(bk[:, None], self.plan.kv_heads, hd)[:, 0],
                                  gather_heads(bv[:, None], self.plan.kv_heads, hd)[:, 0]]).contiguous()
            wo_full = src.weight("o_proj.weight", l, (H, cfg.n_heads * hd), 7)
            wo = gather_head_cols(wo_full, self.plan.q_heads, hd).contiguous()
            wo_scale = ops.ref.quantize_w8(wo_full)[1] if quant != "none" else None
            del wo_full
            gate = src.weight("gate_proj.weight", l, (cfg.intermediate, H), 8)
            up = src.weight("up_proj.weight", l, (cfg.intermediate, H), 9)
            if inter_pad != cfg.intermediate:
                z = torch.zeros(inter_pad - cfg.intermediate, H, dtype=dtype, device=device)
                gate, up = torch.cat([gate, z], 0), torch.cat([up, z], 0)
            wgu = interleave_gate_up(shard_rows(gate, tp, rank), shard_rows(up, tp, rank))
            del gate, up
            down = src.weight("down_proj.weight", l, (H, cfg.intermediate), 10)
            if inter_pad != cfg.intermediate:
                down = torch.cat([down, torch.zeros(H, inter_pad - cfg.intermediate, dtype=dtype,
                                                    device=device)], 1)
            wdown = shard_cols(down, tp, rank)
            down_scale = ops.ref.quantize_w8(down)[1] if quant == "w8a16" else None
            del down
            if quant != "none":
                wqkv, wo = W8Weight(wqkv), W8Weight(wo, wo_scale)
                if quant == "w4a16":
                    wgu, wdown = W4Weight(wgu), W4Weight(wdown)
                else:
                    wgu, wdown = W8Weight(wgu), W8Weight(wdown, down_scale)
            elif tiled:
                wqkv, wo, wgu, wdown = (ops.tile_weight(t) for t in (wqkv, wo, wgu, wdown))
            self.layers.append(dict(
                wqkv=wqkv, bqkv=bqkv, wo=wo, wgu=wgu, wdown=wdown,
                ln1=src.norm("input_layernorm.weight", l, H),
                ln2=src.norm("post_attention_layernorm.weight", l, H)))
        self.embed = src.weight("embed_tokens.weight", -1, (cfg.vocab, H), 900001)
        vocab_pad = -(-cfg.vocab // tp) * tp
        head = src.weight("lm_head.weight", -1, (cfg.vocab, H), 900002)
        if vocab_pad != cfg.vocab:
            head = torch.cat([head, torch.zeros(vocab_pad - cfg.vocab, H, dtype=dtype, device=device)], 0)
        self.vocab_local = vocab_pad // tp
        self.lm_head = shard_rows(head, tp, rank)
        del head
        if quant != "none":
            self.lm_head = W8Weight(self.lm_head)
        elif tiled:
            self.lm_head = ops.tile_weight(self.lm_head)
        self.ln_f = src.norm("norm.weight", -1, H)

    @staticmethod
    def dense(w):
        """The plain [n, k] tensor of a weight, whichever way it is stored."""
        if isinstance(w, (W8Weight, W4Weight)):
            return w.dense()
        return ops.untile_weight(w)

    def nbytes(self):
        n = self.embed.numel() + self.lm_head.numel() + self.ln_f.numel()
        for L in self.layers:
            n += sum(t.numel() for t in L.values() if t is not None)
        return n * self.embed.element_size()


class PagedKV:
    """Paged KV cache: [blocks, nkv_local, block_size, head_dim] per layer, one
    contiguous run of blocks per sequence (block tables are still indirect)."""

    def __init__(self, n_layers, batch, max_len, nkv, hd, device, dtype, block_size=16):
        self.block_size = block_size
        self.blocks_per_seq = -(-max_len // block_size)
        n_blocks = batch * self.blocks_per_seq
        self.k = [torch.zeros(n_blocks, nkv, block_size, hd, dtype=dtype, device=device)
                  for _ in range(n_layers)]
        self.v = [torch.zeros(n_blocks, nkv, block_size, hd, dtype=dtype, device=device)
                  for _ in range(n_layers)]
        self.block_tables = (torch.arange(n_blocks, dtype=torch.int32, device=device)
                             .view(batch, self.blocks_per_seq).contiguous())

    def slots(self, positions_2d, seq_offset=0):
        """positions [batch, s] -> flat slot ids [batch*s] (int32); the rows are
        sequences seq_offset .. seq_offset + batch of the cache."""
        b = torch.arange(positions_2d.shape[0], device=positions_2d.device)[:, None] + seq_offset
        blk = self.block_tables[b, (positions_2d // self.block_size).long()]
        return (blk * self.block_size + positions_2d % self.block_size).to(torch.int32).reshape(-1)


class Qwen2Model:
    def __init__(self, cfg: Qwen2Config, comm: Optional[TPComm] = None, device="cpu",
                 dtype=torch.float32, seed=0, layers=None, quant="none", shard_of=None, source=None):
        """shard_of=(tp, rank): hold that rank's shard of a tp-way split while
        running alone (collectives are no-ops, results are partial sums): the
        per-rank compute of a larger tensor-parallel job, for tuning on one GPU."""
        self.cfg = cfg
        self.comm = comm or TPComm(None)
        self.device, self.dtype = torch.device(device), dtype
        tp, rank = shard_of if shard_of is not None else (self.comm.world, self.comm.rank)
        self.w = Qwen2Weights(cfg, tp, rank, self.device, dtype, seed, layers, quant=quant, source=source)
        self.nq, self.nkv, self.hd = self.w.plan.nq, self.w.plan.nkv, cfg.head_dim
        self.scale = 1.0 / math.sqrt(cfg.head_dim)

    def _run_layers(self, ids, positions, attn_factory, split_k=False):
        """ids [T] int32 -> final normed hidden [T, hidden] (replicated on every rank)."""
        cfg, c, w = self.cfg, self.comm, self.w
        h = ops.embedding(ids, w.embed)
        res = torch.zeros_like(h)
        split_k = split_k and h.is_cuda
        # prefill sizes on the link: the row-parallel linears scatter their output tiles into the
        # owners' staging inboxes from the GEMM epilogue and one kernel finishes the all-reduce
        pushed = (not split_k and h.is_cuda and w.quant == "none" and c.world > 1 and c.use_link
                  and h.shape[0] > 128 and h.shape[0] % c.world == 0 and not w.tiled)
        pending = False  # h holds a partial sum that still needs the all-reduce
        for li, L in enumerate(w.layers):
            if pending:
                normed, res = c.allreduce_rmsnorm(h, res, L["ln1"], cfg.eps)
            else:
                normed, res = ops.rmsnorm(h, L["ln1"], cfg.eps, res)
            if w.quant != "none":
                qkv = qlinear(normed, L["wqkv"], L["bqkv"])
                a = attn_factory(li)(qkv, None)
                h = qlinear(a, L["wo"])
            elif split_k:
                # decode: k-split linears leave fp32 slabs that the next kernel sums
                qkv = ops.linear_split(normed, L["wqkv"])
                if qkv.dtype == torch.float32:
                    a = attn_factory(li)(qkv, L["bqkv"])
                else:
                    if L["bqkv"] is not None:
                        qkv = qkv + L["bqkv"]
                    a = attn_factory(li)(qkv, None)
                h = ops.linear_split(a, L["wo"])
            elif pushed:
                qkv = ops.linear(normed, L["wqkv"], L["bqkv"])
                a = attn_factory(li)(qkv, None)
                h = c.row_parallel(torch.empty_like(res), [(a, L["wo"], None, None, False, 0)])
            else:
                qkv = ops.linear(normed, L["wqkv"], L["bqkv"])
                a = attn_factory(li)(qkv, None)
                h = ops.linear(a, L["wo"])
            if pushed:
                normed, res = ops.rmsnorm(h, L["ln2"], cfg.eps, res)
            else:
                normed, res = c.allreduce_rmsnorm(h, res, L["ln2"], cfg.eps)
            if split_k and w.quant == "none" and ops.k_splits(normed, L["wgu"]) > 1:
                # a gate/up shard with few row tiles fills the SMs only with a k-split;
                # SiLU*mul then runs over the slabs (one small kernel) instead of in the epilogue
                act = ops.silu_mul(ops.linear_split(normed, L["wgu"]), interleaved=True)
            else:
                act = qlinear(normed, L["wgu"], silu_mul=True)
            if pushed:
                h = c.row_parallel(torch.empty_like(res), [(act, L["wdown"], None, None, False, 0)])
                pending = False
            else:
                h = qlinear(act, L["wdown"], split=split_k)
                pending = True
        if pending:
            normed, res = c.allreduce_rmsnorm(h, res, w.ln_f, cfg.eps)
        else:
            normed, res = ops.rmsnorm(h, w.ln_f, cfg.eps, res)
        return normed

    # ---- prefill: dense causal attention, optional KV write ----------------
    def prefill(self, ids_2d, cache: Optional[PagedKV] = None, seq_offset: int = 0):
        """ids [batch, seq] -> final normed hidden [batch*seq, hidden]; with a
        cache, K/V of sequence i go to cache sequence seq_offset + i."""
        batch, seq = ids_2d.shape
        dev = ids_2d.device
        pos2d = torch.arange(seq, device=dev, dtype=torch.int32)[None, :].expand(batch, seq).contiguous()
        positions = pos2d.reshape(-1)
        slots = cache.slots(pos2d, seq_offset) if cache is not None else None
        cu = torch.arange(0, (batch + 1) * seq, seq, device=dev, dtype=torch.int32)
        nq, nkv, hd = self.nq, self.nkv, self.hd

        def attn_factory(li):
            def attn(qkv, bias=None):
                kc = cache.k[li] if cache is not None else None
                vc = cache.v[li] if cache is not None else None
                qkv = ops.rope_kv_write(qkv, positions, slots, kc, vc, nq, nkv, hd,
                                        cache.block_size if cache is not None else 16, self.cfg.theta,
                                        bias)
                T = qkv.shape[0]
                v3 = qkv.view(T, nq + 2 * nkv, hd)
                o = ops.attention(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu, cu, seq,
                                  self.scale, True, max_k=seq)
                return o.reshape(T, nq * hd)
            return attn

        return self._run_layers(ids_2d.reshape(-1).to(torch.int32), positions, attn_factory)

    # ---- decode: one token per sequence against the paged cache ------------
    def decode_hidden(self, ids, positions, slots, ctx_lens, cache: PagedKV, splits=0):
        nq, nkv, hd = self.nq, self.nkv, self.hd

        import os
        fuse = os.environ.get("BL_FUSE_ROPE_ATTN", "0") == "1" and self.device.type == "cuda"

        def attn_factory(li):
            def attn(qkv, bias=None):
                if fuse:
                    # opt-in: RoPE, the KV write and the attention in one launch
                    return ops.rope_attn_decode(qkv, bias, positions, slots, cache.k[li], cache.v[li],
                                                cache.block_tables, ctx_lens, nq, nkv, hd, cache.block_size,
                                                self.cfg.theta, self.scale, splits)
                qkv = ops.rope_kv_write(qkv, positions, slots, cache.k[li], cache.v[li], nq, nkv, hd,
                                        cache.block_size, self.cfg.theta, bias)
                return ops.paged_attn_decode(qkv, cache.k[li], cache.v[li], cache.block_tables,
                                             ctx_lens, nq, nkv, hd, self.scale, splits)
            return attn

        return self._run_layers(ids, positions, attn_factory, split_k=True)

    # ---- decode with one kernel per linear and the collectives folded in ----------
    def dlin_ok(self, tokens):
        """The decode step built from `_C.dlin` kernels: every linear is one cluster split-K
        kernel; o_proj / down store their bf16 partial rows straight into every rank's one-shot
        inbox, and the linear after them (QKV, gate/up) gathers, reduces, adds the residual and
        normalises in its prologue while its weights stream.  Five launches per layer.  Default
        with more than one rank; BL_DLIN=1 selects it on one GPU too (inboxes in local memory),
        BL_DLIN=0 turns it off."""
        import os
        c = self.comm
        mode = os.environ.get("BL_DLIN", DLIN_DEFAULT)
        if mode == "0" or self.device.type != "cuda" or self.w.quant != "none" or self.dtype != torch.bfloat16:
            return False
        if tokens > 64 or self.cfg.hidden % 8 or self.cfg.hidden > 8192 or self.w.tiled:
            return False
        if c.world > 1 and c.no_comm:
            # timing control: same kernels, inboxes in local memory, nothing crosses NVLink
            return mode != "tuned" or c.world in DLIN_TUNED_WORLDS
        if c.world > 1:
            if mode == "tuned" and c.world not in DLIN_TUNED_WORLDS:
                return False
            return bool(c.use_link) and tokens * self.cfg.hidden * 2 <= c.oneshot_max
        return mode == "1"

    def _dlin_buffers(self, tokens):
        key = ("dlin", tokens, self.comm.no_comm)
        if getattr(self, "_dbuf_key", None) != key:
            from .. import load_extension
            H = self.cfg.hidden
            res = torch.zeros(tokens, H, dtype=self.dtype, device=self.device)
            xn = torch.zeros(tokens, H, dtype=self.dtype, device=self.device)
            link = None
            if self.comm.world == 1 or self.comm.no_comm:
                link = load_extension().dlin_local_link(tokens, H, self.device.index or 0)
            self._dbuf, self._dbuf_key = (res, xn, link), key
        return self._dbuf

    def decode_hidden_dlin(self, ids, positions, slots, ctx_lens, cache: PagedKV, splits=0):
        """Same result as decode_hidden (same roundings: each rank's partial row is rounded to
        bf16 before the sum, the sum before the residual add)."""
        from .. import load_extension
        C = load_extension()
        cfg, c, w = self.cfg, self.comm, self.w
        nq, nkv, hd = self.nq, self.nkv, self.hd
        H = cfg.hidden
        res, xn, link = self._dlin_buffers(ids.shape[0])
        # BL_DLIN_PRO=1: the gather + residual + norm runs in the prologue of the linear that needs it
        # (five launches per layer); default: in a small kernel of its own that becomes resident while
        # the row-parallel linear before it is still running (seven launches per layer)
        import os
        in_prologue = os.environ.get("BL_DLIN_PRO", "0") == "1"
        ops.embedding(ids, w.embed, out=res)
        ops.rmsnorm(res, w.layers[0]["ln1"], cfg.eps, out=xn)
        for li, L in enumerate(w.layers):
            ops._count(5 if in_prologue else 7)
            if li == 0 or not in_prologue:
                qkv = C.dlin(xn, L["wqkv"], epi="store", bias=L["bqkv"])
            else:
                qkv = C.dlin(xn, L["wqkv"], pro="gather_norm", epi="store", bias=L["bqkv"], residual=res,
                             gamma=L["ln1"], eps=cfg.eps, link=link)
            a = C.rope_attn_decode(qkv, None, positions, slots, cache.k[li], cache.v[li], cache.block_tables,
                                   ctx_lens, nq, nkv, hd, cfg.theta, self.scale, splits)
            C.dlin(a, L["wo"], epi="push", hidden=H, link=link)
            if in_prologue:
                act = C.dlin(xn, L["wgu"], pro="gather_norm", epi="silu_mul", residual=res, gamma=L["ln2"],
                             eps=cfg.eps, link=link)
            else:
                C.gather_norm(xn, res, L["ln2"], cfg.eps, link=link)
                act = C.dlin(xn, L["wgu"], epi="silu_mul")
            C.dlin(act, L["wdown"], epi="push", hidden=H, link=link)
            if not in_prologue and li + 1 < len(w.layers):
                C.gather_norm(xn, res, w.layers[li + 1]["ln1"], cfg.eps, link=link)
            c.ar_calls += 2 if c.world > 1 else 0
            c.ar_bytes += (2 * xn.numel() * 2) if c.world > 1 else 0
        ops._count()
        C.gather_norm(xn, res, w.ln_f, cfg.eps, link=link)
        return xn

    # ---- decode with the fused tensor-parallel linears -------------------------
    def fused_ok(self, tokens):
        """Row-parallel GEMM->reduce-scatter and all-gather->column-parallel GEMM
        need the link and a token count that splits over the ranks.  They are
        selected with BL_FUSED_LINEAR=1; the default decode path is the k-split
        GEMM followed by the one-hop fused all-reduce+RMSNorm, which measured
        faster at decode sizes (the reduce-scatter/all-gather pair costs two
        flag round trips per half layer, the one-shot all-reduce none)."""
        import os
        c = self.comm
        return (c.world > 1 and c.use_link and tokens % c.world == 0 and tokens <= 256
                and self.device.type == "cuda" and self.w.quant == "none"
                and os.environ.get("BL_FUSED_LINEAR", "0") == "1")

    def _fused_buffers(self, tokens):
        key = ("fused", tokens)
        if getattr(self, "_fbuf_key", None) != key:
            from .. import load_extension
            C = load_extension()
            H, w = self.cfg.hidden, self.comm.world
            smax = 1
            for n, k in ((H, self.nq * self.hd), (H, self.w.inter_local)):
                smax = max(smax, C.gemm_splits(n, k, tokens))
            tpr = tokens // w
            dev = self.device.index or 0
            inbox = C.empty(4 * w * smax * tpr * H, 0, torch.float32)
            gather = C.empty(2 * tokens * H, 0, torch.bfloat16).view(tokens, H)
            inbox.zero_()
            gather.zero_()
            self._fbuf = (inbox, gather, torch.zeros(tpr, H, dtype=self.dtype, device=self.device))
            self._fbuf_key = key
        return self._fbuf

    def decode_hidden_fused(self, ids, positions, slots, ctx_lens, cache: PagedKV, splits=0):
        """Same result as decode_hidden; the residual stream is sharded by tokens:
        o_proj/down push fp32 partial rows to each token's owner from the GEMM
        epilogue, the owner reduces + adds the residual + normalises and stores
        the normed rows into every rank's gather buffer, and the next GEMM waits
        for those rows while its weights are already streaming."""
        from .. import load_extension
        C = load_extension()
        cfg, c, w = self.cfg, self.comm, self.w
        T = ids.shape[0]
        tpr = T // c.world
        nq, nkv, hd = self.nq, self.nkv, self.hd
        inbox, gather, res = self._fused_buffers(T)
        h0 = ops.embedding(ids, w.embed)
        res.copy_(h0[c.rank * tpr:(c.rank + 1) * tpr])
        x, _ = ops.rmsnorm(h0, w.layers[0]["ln1"], cfg.eps)
        gate = 0
        for li, L in enumerate(w.layers):
            qkv = ops.linear_split(x, L["wqkv"], gate_tokens=gate)
            if qkv.dtype == torch.float32:
                qkv = ops.rope_kv_write(qkv, positions, slots, cache.k[li], cache.v[li], nq, nkv, hd,
                                        cache.block_size, cfg.theta, L["bqkv"])
            else:
                if L["bqkv"] is not None:
                    qkv = qkv + L["bqkv"]
                qkv = ops.rope_kv_write(qkv, positions, slots, cache.k[li], cache.v[li], nq, nkv, hd,
                                        cache.block_size, cfg.theta)
            a = ops.paged_attn_decode(qkv, cache.k[li], cache.v[li], cache.block_tables, ctx_lens,
                                      nq, nkv, hd, self.scale, splits)
            ops._count(2)
            units, S = C.tp_gemm_rs(a, *ops._w(L["wo"])[:1], inbox, *ops._w(L["wo"])[1:])
            C.tp_rs_finish(inbox, gather, res, L["ln2"], cfg.eps, T, S, units)
            act = ops.linear(gather, L["wgu"], silu_mul=True, gate_tokens=T)
            nxt = w.layers[li + 1]["ln1"] if li + 1 < len(w.layers) else w.ln_f
            ops._count(2)
            units, S = C.tp_gemm_rs(act, *ops._w(L["wdown"])[:1], inbox, *ops._w(L["wdown"])[1:])
            C.tp_rs_finish(inbox, gather, res, nxt, cfg.eps, T, S, units)
            x, gate = gather, T
            c.ar_calls += 2
        return gather, T

    def logits_local(self, hidden):
        return qlinear(hidden, self.w.lm_head)

    def logits(self, hidden):
        """Full-vocabulary logits (vocab-parallel head + gather)."""
        full = self.comm.all_gather_cols(self.logits_local(hidden))
        return full[:, : self.cfg.vocab]

    def next_tokens(self, hidden, out=None, dlin=False):
        """Greedy next token per row (local arg max + a few bytes per row exchanged).
        dlin: the head may run on the decode-linear kernel; it does when its row tiles fit the GPU
        at once (a vocabulary shard of 149 tiles takes the persistent GEMM two laps of its 148 CTAs)."""
        head = self.w.lm_head
        if (dlin and hidden.is_cuda and isinstance(head, torch.Tensor) and hidden.shape[0] <= 64
                and -(-head.shape[0] // 128) <= 296):
            from .. import load_extension
            ops._count()
            logits = load_extension().dlin(hidden, head, epi="store")
        else:
            logits = self.logits_local(hidden)
        return self.comm.argmax_vocab_parallel(logits, self.w.vocab_local, out)


class DecodeEngine:
    """Greedy decoding with a CUDA-graphed step.

    `prefill(ids)` fills the cache and returns the first generated token;
    `step(ids)` consumes one token per sequence and returns the next one.  On
    CUDA the step is captured once and replayed: the position, slot and
    context-length tensors live on the device and advance inside the graph,
    and the collectives are replay-safe (their expectations are device
    counters).  `step_host` is the end-to-end form: token ids arrive in pinned
    host memory and the result is read back to the host every step.
    """

    def __init__(self, model: Qwen2Model, batch: int, max_len: int, use_graph: bool = True,
                 attn_splits: int = 0):
        self.m = model
        self.batch, self.max_len = batch, max_len
        dev, dt = model.device, model.dtype
        self.cache = PagedKV(len(model.w.layers), batch, max_len, model.nkv, model.hd, dev, dt)
        self.ids = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.positions = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.ctx_lens = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.slots = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.out_ids = torch.zeros(batch, dtype=torch.int32, device=dev)
        self.use_graph = use_graph and dev.type == "cuda"
        self.graph = None
        self.attn_splits = attn_splits
        self.launches_per_step = 0
        if dev.type == "cuda":
            self.h_in = torch.zeros(batch, dtype=torch.int32).pin_memory()
            self.h_out = torch.zeros(batch, dtype=torch.int32).pin_memory()

    def set_context(self, length: int):
        """Declare that every sequence already has `length` tokens in the cache."""
        self.positions.fill_(length)
        self._refresh()

    def _refresh(self):
        c = self.cache
        b = torch.arange(self.batch, device=self.positions.device)
        blk = c.block_tables[b, (self.positions // c.block_size).long()]
        self.slots.copy_(blk * c.block_size + self.positions % c.block_size)
        self.ctx_lens.copy_(self.positions + 1)

    def prefill(self, ids_2d, max_tokens: int = 8192):
        """Run the prompts through the model (a few sequences at a time, at most
        `max_tokens` tokens per pass) and return the first generated token."""
        seq = ids_2d.shape[1]
        per = max(1, max_tokens // seq)
        lasts = []
        for b0 in range(0, self.batch, per):
            part = ids_2d[b0:b0 + per].contiguous()
            hidden = self.m.prefill(part, self.cache, seq_offset=b0)
            lasts.append(hidden.view(part.shape[0], seq, -1)[:, -1])
        last = torch.cat(lasts, 0).contiguous()
        nxt = self.m.next_tokens(last)
        self.set_context(seq)
        return nxt

    def _step_body(self):
        if self.m.dlin_ok(self.batch):
            hidden = self.m.decode_hidden_dlin(self.ids, self.positions, self.slots, self.ctx_lens,
                                               self.cache, self.attn_splits)
            nxt = self.m.next_tokens(hidden, self.out_ids, dlin=True)
        elif self.m.fused_ok(self.batch):
            hidden, gate = self.m.decode_hidden_fused(self.ids, self.positions, self.slots,
                                                      self.ctx_lens, self.cache, self.attn_splits)
            logits = ops.linear(hidden, self.m.w.lm_head, gate_tokens=gate)
            nxt = self.m.comm.argmax_vocab_parallel(logits, self.m.w.vocab_local, self.out_ids)
        else:
            hidden = self.m.decode_hidden(self.ids, self.positions, self.slots, self.ctx_lens,
                                          self.cache, self.attn_splits)
            nxt = self.m.next_tokens(hidden, self.out_ids)
        if nxt is not self.out_ids:
            self.out_ids.copy_(nxt)
        if self.m.device.type == "cuda":
            # one kernel: position, context length, KV slot and next input id
            from .. import load_extension
            ops._count()
            load_extension().decode_advance(self.positions, self.ctx_lens, self.slots,
                                            self.cache.block_tables, self.ids, self.out_ids,
                                            self.cache.block_size)
        else:
            self.ids.copy_(nxt)  # replays feed themselves unless the caller overwrites ids
            self.positions.add_(1)
            self._refresh()

    def capture(self, warmup: int = 2):
        """Warm up (allocator, lazy attributes) and capture the step."""
        if not self.use_graph:
            return
        saved = (self.positions.clone(), self.ids.clone())
        s = torch.cuda.Stream()
        s.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(s):
            for _ in range(warmup):
                self._step_body()
        torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        self.positions.copy_(saved[0])
        self._refresh()
        before = ops.launch_count
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph):
            self._step_body()
        self.launches_per_step = ops.launch_count - before
        # the captured run did not execute; state is as before the capture
        self.positions.copy_(saved[0])
        self.ids.copy_(saved[1])
        self._refresh()
        torch.cuda.synchronize()

    def step(self, ids=None):
        if ids is not None:
            self.ids.copy_(ids)
        if self.graph is not None:
            self.graph.replay()
        else:
            before = ops.launch_count
            self._step_body()
            self.launches_per_step = ops.launch_count - before
        return self.out_ids

    def step_host(self, ids_host):
        """ids_host: pinned int32 [batch] on the host -> pinned int32 [batch] (next tokens)."""
        self.ids.copy_(ids_host, non_blocking=True)
        self.step()
        self.h_out.copy_(self.out_ids, non_blocking=True)
        torch.cuda.current_stream().synchronize()
        return self.h_out
