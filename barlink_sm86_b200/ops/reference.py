# SPDX-License-Identifier: MIT
"""Plain PyTorch fp32 statements of every kernel in this library.

They serve two purposes: they are the oracles that the GPU numerics tests
compare against, and they are the CPU execution path that lets the models and
the tensor-parallel plumbing run (and be tested over gloo) on a machine
without a GPU.  Shapes and argument order match `barlink_sm86_b200.ops`.
"""
import math

import torch


def linear(x, weight, bias=None, residual=None, silu_mul=False, gelu=False):
    """y = x @ weight.T (+ bias) (tanh-GELU) (+ residual); silu_mul: rows of `weight` are
    interleaved (gate, up) pairs and y = silu(gate) * up has half the columns."""
    y = x.float() @ weight.float().t()
    if bias is not None:
        y = y + bias.float()
    if gelu:
        y = torch.nn.functional.gelu(y, approximate="tanh")
    if silu_mul:
        g, u = y[..., 0::2], y[..., 1::2]
        y = torch.nn.functional.silu(g) * u
    if residual is not None:
        y = y + residual.float()
    return y.to(x.dtype)


def rmsnorm(x, gamma, eps, residual=None):
    """Returns (normed, new_residual).  With a residual, x + residual is
    rounded to the storage dtype first and that rounded sum is normalised."""
    if residual is not None:
        s = (x.float() + residual.float()).to(x.dtype)
    else:
        s = x
    f = s.float()
    var = f.pow(2).mean(-1, keepdim=True)
    n = (f * torch.rsqrt(var + eps)).to(x.dtype)
    out = (n.float() * gamma.float()).to(x.dtype)
    return out, (s if residual is not None else None)


def _rope_angles(positions, dim, theta):
    inv = theta ** (-torch.arange(0, dim, 2, dtype=torch.float32, device=positions.device) / dim)
    ang = positions.float()[:, None] * inv[None, :]
    return ang.cos(), ang.sin()


def rope(x, positions, theta, axes=1):
    """Rotate-half RoPE on x [rows, heads, hd].  axes=2: positions [rows, 2]
    and each half of hd is rotated by its own coordinate."""
    rows, heads, hd = x.shape
    out = x.float().clone()
    sub = hd // axes
    pos = positions.view(rows, axes)
    for a in range(axes):
        cos, sin = _rope_angles(pos[:, a], sub, theta)
        seg = out[..., a * sub:(a + 1) * sub]
        x1, x2 = seg[..., : sub // 2], seg[..., sub // 2:]
        c, s = cos[:, None, :], sin[:, None, :]
        out[..., a * sub:(a + 1) * sub] = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], -1)
    return out.to(x.dtype)


def qknorm_rope(qkv, gq, gk, positions, heads, eps=1e-6, theta=1e4, axes=2):
    """In place: per-head RMSNorm of the q and k heads at the start of each row
    of qkv [rows, width] (head_dim 128), then RoPE with `axes` coordinates."""
    rows = qkv.shape[0]
    qk = qkv[:, : 2 * heads * 128].reshape(rows, 2 * heads, 128).float()
    for lo, g in ((0, gq), (heads, gk)):
        if g is None:
            continue
        seg = qk[:, lo:lo + heads]
        n = (seg * torch.rsqrt(seg.pow(2).mean(-1, keepdim=True) + eps)).to(qkv.dtype).float()
        qk[:, lo:lo + heads] = n * g.float()
    rot = rope(qk.to(qkv.dtype), positions, theta, axes)
    qkv[:, : 2 * heads * 128] = rot.reshape(rows, 2 * heads * 128)
    return qkv


def layernorm_modulate(x, shift, scale, rows_per_batch, eps=1e-6):
    rows = x.numel() // x.shape[-1]
    f = x.reshape(rows, -1).float()
    n = torch.nn.functional.layer_norm(f, (f.shape[-1],), eps=eps)
    b = torch.arange(rows, device=x.device) // rows_per_batch
    out = n * (1.0 + scale.float()[b]) + shift.float()[b]
    return out.to(x.dtype).view_as(x)


def gate_residual(x, y, gate, rows_per_batch):
    rows = x.numel() // x.shape[-1]
    b = torch.arange(rows, device=x.device) // rows_per_batch
    x.copy_((x.reshape(rows, -1).float() + gate.float()[b] * y.reshape(rows, -1).float()).to(x.dtype).view_as(x))
    return x


def rope_kv_write(qkv, positions, slots, k_cache, v_cache, nq, nkv, hd, block_size, theta):
    """In place: rotate q and k inside qkv [rows, (nq+2nkv)*hd]; store k, v at
    slot (= block * block_size + offset) of caches [blocks, nkv, block_size, hd]."""
    rows = qkv.shape[0]
    v3 = qkv.view(rows, nq + 2 * nkv, hd)
    v3[:, : nq + nkv] = rope(v3[:, : nq + nkv], positions, theta)
    if slots is not None:
        for r in range(rows):
            s = int(slots[r])
            if s < 0:
                continue
            blk, off = divmod(s, block_size)
            k_cache[blk, :, off, :] = v3[r, nq:nq + nkv]
            v_cache[blk, :, off, :] = v3[r, nq + nkv:]
    return qkv


def silu_mul(gate_up, interleaved=False):
    if gate_up.dtype == torch.float32 and gate_up.dim() == 3:  # k-split slabs: summed first
        g, u = gate_up.sum(0)[..., 0::2], gate_up.sum(0)[..., 1::2]
        return (torch.nn.functional.silu(g) * u).to(torch.bfloat16)
    f = gate_up.float()
    if interleaved:
        g, u = f[..., 0::2], f[..., 1::2]
    else:
        h = f.shape[-1] // 2
        g, u = f[..., :h], f[..., h:]
    return (torch.nn.functional.silu(g) * u).to(gate_up.dtype)


def embedding(ids, table, vocab_lo=0):
    out = torch.zeros(ids.numel(), table.shape[1], dtype=table.dtype, device=table.device)
    loc = ids.long() - vocab_lo
    ok = (loc >= 0) & (loc < table.shape[0])
    out[ok] = table[loc[ok]]
    return out


def argmax(logits, offset=0):
    val, idx = logits.float().max(-1)
    return (idx + offset).to(torch.int32), val


def paged_attn_decode(q, k_cache, v_cache, block_tables, ctx_lens, nq, nkv, hd, scale):
    """q [batch, >= nq*hd] (first nq*hd columns are the query heads)."""
    batch = q.shape[0]
    bs = k_cache.shape[2]
    G = nq // nkv
    out = torch.zeros(batch, nq * hd, dtype=q.dtype, device=q.device)
    for b in range(batch):
        n = int(ctx_lens[b])
        if n == 0:
            continue
        nb = (n + bs - 1) // bs
        blks = block_tables[b, :nb].long()
        k = k_cache[blks].permute(1, 0, 2, 3).reshape(nkv, nb * bs, hd)[:, :n].float()
        v = v_cache[blks].permute(1, 0, 2, 3).reshape(nkv, nb * bs, hd)[:, :n].float()
        qq = q[b, : nq * hd].view(nkv, G, hd).float()
        s = torch.einsum("hgd,htd->hgt", qq, k) * scale
        p = torch.softmax(s, -1)
        o = torch.einsum("hgt,htd->hgd", p, v)
        out[b] = o.reshape(nq * hd).to(q.dtype)
    return out


def attention(q, k, v, cu_q, cu_k, scale, causal):
    """Dense attention over packed sequences.  q [tq, nq, hd], k/v [tk, nkv, hd];
    cu_* are cumulative lengths (batch + 1).  causal aligns the last query of a
    sequence with its last key."""
    nq, nkv = q.shape[1], k.shape[1]
    G = nq // nkv
    out = torch.zeros_like(q)
    for b in range(len(cu_q) - 1):
        q0, q1, k0, k1 = int(cu_q[b]), int(cu_q[b + 1]), int(cu_k[b]), int(cu_k[b + 1])
        qq = q[q0:q1].float().permute(1, 0, 2)
        kk = k[k0:k1].float().permute(1, 0, 2).repeat_interleave(G, 0)
        vv = v[k0:k1].float().permute(1, 0, 2).repeat_interleave(G, 0)
        s = qq @ kk.transpose(1, 2) * scale
        if causal:
            lq, lk = q1 - q0, k1 - k0
            i = torch.arange(lq, device=q.device)[:, None] + (lk - lq)
            j = torch.arange(lk, device=q.device)[None, :]
            s = s.masked_fill(j > i, float("-inf"))
        o = torch.softmax(s, -1) @ vv
        out[q0:q1] = o.permute(1, 0, 2).to(q.dtype)
    return out


def quantize_w8(weight):
    """Symmetric per-output-channel int8: returns (wq int8 [n, k], scale bf16 [n])."""
    w = weight.float()
    amax = w.abs().amax(1).clamp_min(1e-12)
    scale = (amax / 127.0).to(torch.bfloat16)
    wq = torch.round(w / scale.float()[:, None]).clamp(-127, 127).to(torch.int8)
    return wq, scale


def w8_dequant(wq, scale):
    """int8 [n, k] with per-channel scales [n] or per-group scales [n, k/group] -> fp32 [n, k]."""
    if scale.dim() == 1:
        return wq.float() * scale.float()[:, None]
    n, k = wq.shape
    g = scale.shape[1]
    return (wq.float().view(n, g, k // g) * scale.float()[:, :, None]).view(n, k)


def quantize_w8_grouped(weight, group=128):
    """Symmetric int8 with one scale per (output channel, group of `group` inputs): the
    granularity of the reference's kernel (torch_ext/barlink_sm86/w8a16.cu:13-24)."""
    w = weight.float()
    n, k = w.shape
    wg = w.view(n, k // group, group)
    scale = (wg.abs().amax(2).clamp_min(1e-12) / 127.0).to(torch.bfloat16)
    wq = torch.round(wg / scale.float()[:, :, None]).clamp(-127, 127).to(torch.int8).view(n, k)
    return wq, scale


def w8a16_linear(x, wq, scale, bias=None, silu_mul=False):
    """y = x @ (wq * scale).T: bf16 activations, int8 weights widened exactly to
    bf16, fp32 accumulation; scale per output channel [n] (applied at the end) or
    per group [n, k/group] (applied to the weights)."""
    if scale.dim() == 2:
        y = x.float() @ w8_dequant(wq, scale).t()
    else:
        y = (x.float() @ wq.float().t()) * scale.float()[None, :]
    if bias is not None:
        y = y + bias.float()
    if silu_mul:
        g, u = y[..., 0::2], y[..., 1::2]
        y = torch.nn.functional.silu(g) * u
    return y.to(x.dtype)


def w8a8_dynamic_linear(x, wq, scale, bias=None, silu_mul=False):
    """The int8-activation form of `w8a16_linear`: per-token scale amax / 127, activations rounded to
    int8, exact integer products, result * scale[n] * xs[m] (torch_ext/barlink_sm86/w8a16.cu:37-150
    of the reference, with per-channel weight scales)."""
    xf = x.float()
    xs = (xf.abs().amax(dim=1) / 127.0).clamp_min(1e-12)
    xq = torch.round(xf / xs[:, None]).clamp(-127, 127)
    if scale.dim() == 2:
        # per-group weight scales: integer sums per group, scaled and added in fp32 (w8a16.cu:119-142 there)
        n, groups = scale.shape
        gk = wq.shape[1] // groups
        part = torch.einsum("mgk,ngk->mng", xq.double().view(-1, groups, gk), wq.double().view(n, groups, gk))
        y = (part * scale.double()[None, :, :]).sum(-1).float() * xs[:, None]
    else:
        y = (xq.double() @ wq.double().t()).float() * scale.float()[None, :] * xs[:, None]
    if bias is not None:
        y = y + bias.float()
    if silu_mul:
        g, u = y[..., 0::2], y[..., 1::2]
        y = torch.nn.functional.silu(g) * u
    return y.to(x.dtype)


def allreduce_rmsnorm(parts, residual, gamma, eps):
    """What the fused kernel computes on every rank, given all ranks' inputs:
    sum in fp32 in rank order, round, add the residual, round, normalise."""
    acc = torch.zeros_like(parts[0], dtype=torch.float32)
    for p in parts:
        acc = acc + p.float()
    s = acc.to(parts[0].dtype)
    if residual is not None:
        s = (s.float() + residual.float()).to(s.dtype)
    normed, _ = rmsnorm(s, gamma, eps)
    return normed, s


def default_scale(hd):
    return 1.0 / math.sqrt(hd)


def pack_int4(weight, group_size=128):
    """[n, k] weight -> GPTQ-v1 tensors (qweight int32 [k/8, n], scales fp16
    [k/group, n], qzeros int32 [k/group, n/8]), symmetric with zero point 8:
    the format of the reference's Int4Linear (demos/qwen_tp/int4linear.py:47-69)."""
    w = weight.float()
    n, k = w.shape
    assert k % group_size == 0 and n % 8 == 0 and k % 8 == 0
    groups = k // group_size
    wg = w.reshape(n, groups, group_size)
    scale = (wg.abs().amax(2) / 7.0).clamp(min=1e-8).half()            # [n, groups], as stored
    q = torch.round(wg / scale.float()[..., None] + 8.0).clamp(0, 15).to(torch.int64).reshape(n, k)
    qk = q.reshape(n, k // 8, 8)
    qw = sum(qk[..., j] << (4 * j) for j in range(8))
    qw = ((qw + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32).t().contiguous()
    z = torch.full((groups, n // 8, 8), 8, dtype=torch.int64, device=w.device)
    qz = sum(z[..., j] << (4 * j) for j in range(8))
    qz = ((qz + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32).contiguous()
    return qw, scale.t().contiguous(), qz


def w4_dequant(qweight, scales, qzeros, group_size=128):
    """GPTQ-v1 tensors -> fp32 [n, k]."""
    k, n = qweight.shape[0] * 8, qweight.shape[1]
    w = qweight.t().long() & 0xFFFFFFFF
    nib = torch.stack([(w >> (4 * j)) & 0xF for j in range(8)], 2).reshape(n, k)
    zz = qzeros.long() & 0xFFFFFFFF
    z = torch.stack([(zz >> (4 * j)) & 0xF for j in range(8)], 2).reshape(-1, n)     # [groups, n]
    z = z.repeat_interleave(group_size, 0)[:k].t()
    sc = scales.float().repeat_interleave(group_size, 0)[:k].t()
    return (nib - z).float() * sc


def w4a16_linear(x, qweight, scales, qzeros, group_size=128):
    return (x.float() @ w4_dequant(qweight, scales, qzeros, group_size).t()).to(x.dtype)
