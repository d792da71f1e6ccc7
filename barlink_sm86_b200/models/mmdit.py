# SPDX-License-Identifier: MIT
"""Flux-style MMDiT (multimodal diffusion transformer) with tensor parallelism.

Architecture: `double_blocks` two-stream blocks (image and text tokens have
their own weights and meet in one joint attention), then `single_blocks`
one-stream blocks over the concatenated sequence; adaLN modulation from a
timestep embedding, per-head RMSNorm on q and k, RoPE over two position axes,
tanh-GELU MLP of ratio 4.  The default configuration is the 12B shape
(19 + 38 blocks, hidden 3072, 24 heads of 128).

The reference runs this family through diffusers with a `_tp_plan` that makes
the qkv / MLP-in projections column-parallel and the out projections
row-parallel with an all-reduce hook (demos/flux2_tp/worker.py:60-150).  Here
the same split is explicit: every rank holds `heads / tp` heads and
`mlp / tp` hidden features, the two row-parallel outputs of a block are summed
by the link's all-reduce kernel (one call per sub-layer, both streams in one
buffer), and every matrix product is the tcgen05 GEMM with bias / GELU /
residual in its epilogue.  Elementwise work is three kernels: LayerNorm +
modulate, q/k-norm + RoPE, gated residual.

The same class runs on CPU tensors (fp32 statements of each op), which is the
oracle of the GPU test and lets the tensor-parallel split be tested over gloo.
"""
import math
from dataclasses import dataclass

import torch

from .. import ops
from ..parallel import TPComm


@dataclass
class MMDiTConfig:
    hidden: int = 3072
    heads: int = 24
    head_dim: int = 128
    mlp_ratio: int = 4
    double_blocks: int = 19
    single_blocks: int = 38
    in_channels: int = 64
    txt_dim: int = 4096
    time_dim: int = 256
    rope_theta: float = 10000.0
    eps: float = 1e-6

    @classmethod
    def flux_12b(cls):
        return cls()

    @classmethod
    def tiny(cls, hidden=256, heads=2, double_blocks=2, single_blocks=2, in_channels=64, txt_dim=128):
        return cls(hidden=hidden, heads=heads, double_blocks=double_blocks, single_blocks=single_blocks,
                   in_channels=in_channels, txt_dim=txt_dim)

    @property
    def mlp(self):
        return self.hidden * self.mlp_ratio

    def params(self):
        h, m = self.hidden, self.mlp
        attn = self.heads * self.head_dim
        stream = 6 * h * h + 3 * attn * h + attn * h + 2 * h * m
        single = 3 * h * h + (3 * attn + m) * h + (attn + m) * h
        return (self.double_blocks * 2 * stream + self.single_blocks * single + self.in_channels * h * 2
                + self.txt_dim * h + self.time_dim * h + h * h + 2 * h * h)


class _Gen:
    """Deterministic weight source: every tensor is drawn in full from a
    generator keyed by its name, then cut, so all ranks agree on the unsharded
    model without talking to each other."""

    def __init__(self, seed, device, dtype, gen_device):
        self.seed, self.device, self.dtype, self.gen_device = seed, device, dtype, gen_device
        self.count = 0

    def __call__(self, rows, cols, std=None):
        g = torch.Generator(device=self.gen_device)
        g.manual_seed(self.seed * 1000003 + self.count)
        self.count += 1
        std = std if std is not None else 1.0 / math.sqrt(cols)
        w = torch.randn(rows, cols, generator=g, device=self.gen_device, dtype=torch.float32) * std
        return w.to(self.dtype)

    def vec(self, n, std=0.02, mean=0.0):
        g = torch.Generator(device=self.gen_device)
        g.manual_seed(self.seed * 1000003 + self.count)
        self.count += 1
        return (torch.randn(n, generator=g, device=self.gen_device, dtype=torch.float32) * std + mean).to(self.dtype)


def _head_rows(w, heads, hd, tp, rank):
    """Rows of a fused [q | k | v] projection (3 * heads * hd rows) that belong
    to this rank's heads, again ordered [q | k | v]."""
    per = heads // tp
    parts = []
    for j in range(3):
        lo = (j * heads + rank * per) * hd
        parts.append(w[lo:lo + per * hd])
    return torch.cat(parts, 0)


def _rows(w, tp, rank):
    per = w.shape[0] // tp
    return w[rank * per:(rank + 1) * per]


def _cols(w, tp, rank):
    per = w.shape[1] // tp
    return w[:, rank * per:(rank + 1) * per]


class MMDiTWeights:
    """Random-init weights of the architecture, sharded for (tp, rank)."""

    def __init__(self, cfg, device="cuda", dtype=torch.bfloat16, seed=0, tp=1, rank=0, gen_device=None):
        if cfg.heads % tp or cfg.mlp % tp:
            raise ValueError("tp=%d must divide %d heads and %d MLP features" % (tp, cfg.heads, cfg.mlp))
        if cfg.head_dim != 128:
            raise ValueError("the attention and q/k-norm kernels are built for head_dim 128")
        if gen_device is None:
            gen_device = "cpu" if cfg.params() < 3e8 else device
        gen = _Gen(seed, device, dtype, gen_device)
        h, hd, nh = cfg.hidden, cfg.head_dim, cfg.heads
        attn = nh * hd
        dev = lambda t: t.contiguous().to(device)
        first = rank == 0  # biases of row-parallel layers are added once
        zero_if = lambda b: b if first else torch.zeros_like(b)

        self.cfg, self.tp, self.rank = cfg, tp, rank
        self.img_in_w, self.img_in_b = dev(gen(h, cfg.in_channels)), dev(gen.vec(h))
        self.txt_in_w, self.txt_in_b = dev(gen(h, cfg.txt_dim)), dev(gen.vec(h))
        self.t1_w, self.t1_b = dev(gen(h, cfg.time_dim)), dev(gen.vec(h))
        self.t2_w, self.t2_b = dev(gen(h, h)), dev(gen.vec(h))

        def stream():
            s = {}
            s["mod_w"], s["mod_b"] = dev(gen(6 * h, h, 0.5 / math.sqrt(h))), dev(gen.vec(6 * h))
            s["qkv_w"] = dev(_head_rows(gen(3 * attn, h), nh, hd, tp, rank))
            s["qkv_b"] = dev(_head_rows(gen.vec(3 * attn)[:, None], nh, hd, tp, rank)[:, 0])
            s["gq"], s["gk"] = dev(gen.vec(hd, 0.05, 1.0)), dev(gen.vec(hd, 0.05, 1.0))
            s["proj_w"] = dev(_cols(gen(h, attn), tp, rank))
            s["proj_b"] = dev(zero_if(gen.vec(h)))
            s["fc1_w"], s["fc1_b"] = dev(_rows(gen(cfg.mlp, h), tp, rank)), dev(_rows(gen.vec(cfg.mlp), tp, rank))
            s["fc2_w"] = dev(_cols(gen(h, cfg.mlp), tp, rank))
            s["fc2_b"] = dev(zero_if(gen.vec(h)))
            return s

        self.double = [{"img": stream(), "txt": stream()} for _ in range(cfg.double_blocks)]
        self.single = []
        for _ in range(cfg.single_blocks):
            s = {}
            s["mod_w"], s["mod_b"] = dev(gen(3 * h, h, 0.5 / math.sqrt(h))), dev(gen.vec(3 * h))
            s["qkv_w"] = dev(_head_rows(gen(3 * attn, h), nh, hd, tp, rank))
            s["qkv_b"] = dev(_head_rows(gen.vec(3 * attn)[:, None], nh, hd, tp, rank)[:, 0])
            s["mlp_w"], s["mlp_b"] = dev(_rows(gen(cfg.mlp, h), tp, rank)), dev(_rows(gen.vec(cfg.mlp), tp, rank))
            s["gq"], s["gk"] = dev(gen.vec(hd, 0.05, 1.0)), dev(gen.vec(hd, 0.05, 1.0))
            w2 = gen(h, attn + cfg.mlp)
            s["out_attn_w"] = dev(_cols(w2[:, :attn], tp, rank))
            s["out_mlp_w"] = dev(_cols(w2[:, attn:], tp, rank))
            s["out_b"] = dev(zero_if(gen.vec(h)))
            self.single.append(s)
        self.final_mod_w, self.final_mod_b = dev(gen(2 * h, h, 0.5 / math.sqrt(h))), dev(gen.vec(2 * h))
        self.final_w, self.final_b = dev(gen(cfg.in_channels, h)), dev(gen.vec(cfg.in_channels))

    def nbytes(self):
        total = 0
        stack = [self.__dict__]
        while stack:
            o = stack.pop()
            for v in (o.values() if isinstance(o, dict) else o):
                if isinstance(v, torch.Tensor):
                    total += v.numel() * v.element_size()
                elif isinstance(v, (dict, list)):
                    stack.append(v)
        return total


def timestep_embedding(t, dim, max_period=10000.0):
    """Sinusoidal embedding of t [batch] (floats in [0, 1], scaled by 1000)."""
    half = dim // 2
    freqs = torch.exp(-math.log(max_period) * torch.arange(half, dtype=torch.float32, device=t.device) / half)
    args = t.float()[:, None] * 1000.0 * freqs[None]
    return torch.cat([torch.cos(args), torch.sin(args)], -1)


def grid_positions(height, width, device):
    """int32 [height*width, 2] (row, column) positions of a latent grid."""
    ys, xs = torch.meshgrid(torch.arange(height), torch.arange(width), indexing="ij")
    return torch.stack([ys.reshape(-1), xs.reshape(-1)], -1).to(torch.int32).to(device)


class MMDiTModel:
    def __init__(self, cfg, weights, comm=None):
        self.cfg, self.w = cfg, weights
        self.comm = comm if comm is not None else TPComm.single()
        if self.comm.world != weights.tp:
            raise ValueError("weights are cut for tp=%d but the communicator has %d ranks"
                             % (weights.tp, self.comm.world))
        self.hl = cfg.heads // weights.tp
        self.scale = 1.0 / math.sqrt(cfg.head_dim)

    # ---- pieces ------------------------------------------------------------
    def _attention(self, qkv, batch, seq):
        """qkv [batch*seq, >= 3*hl*128] with rows laid out [q | k | v]."""
        hl, hd = self.hl, self.cfg.head_dim
        v3 = qkv[:, : 3 * hl * hd].unflatten(1, (3 * hl, hd))
        cu = torch.arange(0, (batch + 1) * seq, seq, dtype=torch.int32, device=qkv.device)
        o = ops.attention(v3[:, :hl], v3[:, hl:2 * hl], v3[:, 2 * hl:], cu, cu, seq, self.scale, False, max_k=seq)
        return o.reshape(batch * seq, hl * hd)

    def _double(self, blk, h, nt, ni, batch, svec, pos_t, pos_i):
        """h: [batch*nt + batch*ni, hidden], text rows first (stream-major)."""
        cfg, hl, hd = self.cfg, self.hl, self.cfg.head_dim
        H = cfg.hidden
        rt, ri = batch * nt, batch * ni
        ht, hi = h[:rt], h[rt:]
        L = nt + ni
        mods = {}
        for name in ("txt", "img"):
            m = ops.linear(svec, blk[name]["mod_w"], blk[name]["mod_b"])
            mods[name] = [m[:, j * H:(j + 1) * H] for j in range(6)]

        W = 3 * hl * hd
        joint = torch.empty(batch * L, W, dtype=h.dtype, device=h.device)
        for name, x, n, pos, lo in (("txt", ht, nt, pos_t, 0), ("img", hi, ni, pos_i, nt)):
            s, (sh, sc) = blk[name], mods[name][0:2]
            xm = ops.layernorm_modulate(x, sh, sc, n, cfg.eps)
            if batch == 1:
                qkv = ops.linear(xm, s["qkv_w"], s["qkv_b"], out=joint[lo:lo + n])
                ops.qknorm_rope(qkv, s["gq"], s["gk"], pos, hl, cfg.eps, cfg.rope_theta, 2)
            else:
                qkv = ops.linear(xm, s["qkv_w"], s["qkv_b"])
                ops.qknorm_rope(qkv, s["gq"], s["gk"], pos, hl, cfg.eps, cfg.rope_theta, 2)
                joint.view(batch, L, W)[:, lo:lo + n] = qkv.view(batch, n, W)
        att = self._attention(joint, batch, L)
        if batch == 1:
            at, ai = att[:nt], att[nt:]
        else:
            a3 = att.view(batch, L, hl * hd)
            at, ai = a3[:, :nt].reshape(rt, hl * hd), a3[:, nt:].reshape(ri, hl * hd)
        o = torch.empty_like(h)
        self.comm.row_parallel(o, [(at, blk["txt"]["proj_w"], blk["txt"]["proj_b"], None, False, 0),
                                   (ai, blk["img"]["proj_w"], blk["img"]["proj_b"], None, False, rt)])
        ops.gate_residual(ht, o[:rt], mods["txt"][2], nt)
        ops.gate_residual(hi, o[rt:], mods["img"][2], ni)

        o = torch.empty_like(h)
        parts = []
        for name, x, n, lo in (("txt", ht, nt, 0), ("img", hi, ni, rt)):
            s, (sh, sc) = blk[name], mods[name][3:5]
            xm = ops.layernorm_modulate(x, sh, sc, n, cfg.eps)
            f = ops.linear(xm, s["fc1_w"], s["fc1_b"], gelu=True)
            parts.append((f, s["fc2_w"], s["fc2_b"], None, False, lo))
        self.comm.row_parallel(o, parts)
        ops.gate_residual(ht, o[:rt], mods["txt"][5], nt)
        ops.gate_residual(hi, o[rt:], mods["img"][5], ni)

    def _single(self, s, x, L, batch, svec, pos):
        cfg, hl, hd = self.cfg, self.hl, self.cfg.head_dim
        H = cfg.hidden
        m = ops.linear(svec, s["mod_w"], s["mod_b"])
        sh, sc, gt = m[:, :H], m[:, H:2 * H], m[:, 2 * H:]
        xm = ops.layernorm_modulate(x, sh, sc, L, cfg.eps)
        qkv = ops.linear(xm, s["qkv_w"], s["qkv_b"])
        ops.qknorm_rope(qkv, s["gq"], s["gk"], pos, hl, cfg.eps, cfg.rope_theta, 2)
        f = ops.linear(xm, s["mlp_w"], s["mlp_b"], gelu=True)
        att = self._attention(qkv, batch, L)
        o_attn = ops.linear(att, s["out_attn_w"], s["out_b"])
        o = torch.empty_like(o_attn)
        self.comm.row_parallel(o, [(f, s["out_mlp_w"], None, o_attn, False, 0)])
        ops.gate_residual(x, o, gt, L)

    # ---- forward -----------------------------------------------------------
    def forward(self, img, txt, timestep, img_pos, txt_pos=None):
        """img [batch, ni, in_channels], txt [batch, nt, txt_dim], timestep
        [batch]; img_pos int32 [ni, 2] (txt_pos defaults to zeros).  Returns
        the predicted velocity [batch, ni, in_channels]."""
        cfg, w = self.cfg, self.w
        batch, ni, _ = img.shape
        nt = txt.shape[1]
        dev, dt = img.device, w.img_in_w.dtype
        H, L = cfg.hidden, nt + ni
        if txt_pos is None:
            txt_pos = torch.zeros(nt, 2, dtype=torch.int32, device=dev)
        pos_t = txt_pos.repeat(batch, 1).contiguous()
        pos_i = img_pos.repeat(batch, 1).contiguous()
        pos_j = torch.cat([txt_pos, img_pos], 0).repeat(batch, 1).contiguous()

        temb = timestep_embedding(timestep, cfg.time_dim).to(dt)
        v = ops.linear(temb, w.t1_w, w.t1_b)
        v = torch.nn.functional.silu(v.float()).to(dt)
        vec = ops.linear(v, w.t2_w, w.t2_b)
        svec = torch.nn.functional.silu(vec.float()).to(dt)

        rt = batch * nt
        h = torch.empty(batch * L, H, dtype=dt, device=dev)
        ops.linear(txt.reshape(rt, cfg.txt_dim).to(dt), w.txt_in_w, w.txt_in_b, out=h[:rt])
        ops.linear(img.reshape(batch * ni, cfg.in_channels).to(dt), w.img_in_w, w.img_in_b, out=h[rt:])
        for blk in w.double:
            self._double(blk, h, nt, ni, batch, svec, pos_t, pos_i)

        if batch == 1:
            x = h
        else:
            x = torch.empty_like(h)
            x3 = x.view(batch, L, H)
            x3[:, :nt] = h[:rt].view(batch, nt, H)
            x3[:, nt:] = h[rt:].view(batch, ni, H)
        for s in w.single:
            self._single(s, x, L, batch, svec, pos_j)

        xi = x.view(batch, L, H)[:, nt:].reshape(batch * ni, H)
        m = ops.linear(svec, w.final_mod_w, w.final_mod_b)
        xf = ops.layernorm_modulate(xi, m[:, :H], m[:, H:], ni, cfg.eps)
        out = ops.linear(xf, w.final_w, w.final_b)
        return out.view(batch, ni, cfg.in_channels)

    def flops_per_forward(self, batch, ni, nt):
        """Dense matrix-product and attention FLOPs of one forward, whole model."""
        cfg = self.cfg
        L = ni + nt
        attn = cfg.heads * cfg.head_dim
        stream = 2 * cfg.hidden * (3 * attn + attn + 2 * cfg.mlp)
        single = 2 * cfg.hidden * (3 * attn + cfg.mlp + attn + cfg.mlp)
        gemm = batch * L * (cfg.double_blocks * stream + cfg.single_blocks * single)
        att = batch * 4 * L * L * attn * (cfg.double_blocks + cfg.single_blocks)
        return gemm + att


def denoise(model, img, txt, img_pos, steps, txt_pos=None):
    """Rectified-flow Euler sampler: `steps` forwards from t = 1 to t = 0."""
    batch = img.shape[0]
    ts = torch.linspace(1.0, 0.0, steps + 1)
    x = img
    for i in range(steps):
        t = torch.full((batch,), float(ts[i]), device=img.device)
        vel = model.forward(x, txt, t, img_pos, txt_pos)
        x = (x.float() + (float(ts[i + 1]) - float(ts[i])) * vel.float()).to(img.dtype)
    return x
