# SPDX-License-Identifier: MIT
"""The fp32 oracles (`ops/reference.py`) against PyTorch's own operators: the GPU
tests compare kernels to these statements, so the statements themselves are checked
against independent implementations here."""
import math

import pytest
import torch
import torch.nn.functional as F

from barlink_sm86_b200.ops import reference as ref


def test_rmsnorm_matches_torch():
    g = torch.Generator().manual_seed(0)
    x, r, w = torch.randn(5, 64, generator=g), torch.randn(5, 64, generator=g), torch.rand(64, generator=g) + 0.5
    out, res = ref.rmsnorm(x, w, 1e-6, r)
    assert torch.allclose(res, x + r)
    assert torch.allclose(out, F.rms_norm(x + r, (64,), w, 1e-6), atol=1e-5)
    out2, none = ref.rmsnorm(x, w, 1e-6)
    assert none is None and torch.allclose(out2, F.rms_norm(x, (64,), w, 1e-6), atol=1e-5)


@pytest.mark.parametrize("causal", [False, True])
def test_attention_matches_sdpa(causal):
    g = torch.Generator().manual_seed(1)
    nq, nkv, hd = 6, 2, 32
    lens = [7, 13]
    q = torch.randn(sum(lens), nq, hd, generator=g)
    k = torch.randn(sum(lens), nkv, hd, generator=g)
    v = torch.randn(sum(lens), nkv, hd, generator=g)
    cu = torch.tensor([0, 7, 20], dtype=torch.int32)
    got = ref.attention(q, k, v, cu, cu, 1 / math.sqrt(hd), causal)
    for b, (lo, hi) in enumerate(((0, 7), (7, 20))):
        qq = q[lo:hi].permute(1, 0, 2)[None]
        kk = k[lo:hi].permute(1, 0, 2)[None]
        vv = v[lo:hi].permute(1, 0, 2)[None]
        want = F.scaled_dot_product_attention(qq, kk, vv, is_causal=causal, enable_gqa=True)[0].permute(1, 0, 2)
        assert torch.allclose(got[lo:hi], want, atol=1e-5), b


def test_paged_decode_attention_matches_dense_attention():
    g = torch.Generator().manual_seed(2)
    nq, nkv, hd, bs, batch = 4, 2, 16, 4, 3
    ctx = torch.tensor([5, 1, 12], dtype=torch.int32)
    nblk = 16
    kc, vc = torch.randn(nblk, nkv, bs, hd, generator=g), torch.randn(nblk, nkv, bs, hd, generator=g)
    bt = torch.randperm(nblk, generator=g)[:12].view(batch, 4).to(torch.int32)
    q = torch.randn(batch, nq * hd, generator=g)
    got = ref.paged_attn_decode(q, kc, vc, bt, ctx, nq, nkv, hd, 0.25)
    for b in range(batch):
        n = int(ctx[b])
        toks_k = torch.cat([kc[int(bt[b, j])] for j in range(4)], 1)[:, :n]   # [nkv, n, hd]
        toks_v = torch.cat([vc[int(bt[b, j])] for j in range(4)], 1)[:, :n]
        want = F.scaled_dot_product_attention(q[b].view(1, nq, 1, hd), toks_k[None], toks_v[None], scale=0.25,
                                              enable_gqa=True).reshape(nq * hd)
        assert torch.allclose(got[b], want, atol=1e-5), b


def test_layernorm_modulate_gate_residual_and_gelu():
    g = torch.Generator().manual_seed(3)
    x = torch.randn(6, 32, generator=g)
    mod = torch.randn(2, 96, generator=g) * 0.3
    sh, sc, gt = mod[:, :32], mod[:, 32:64], mod[:, 64:]
    got = ref.layernorm_modulate(x, sh, sc, 3)
    ln = F.layer_norm(x, (32,), eps=1e-6)
    want = torch.cat([ln[:3] * (1 + sc[0]) + sh[0], ln[3:] * (1 + sc[1]) + sh[1]])
    assert torch.allclose(got, want, atol=1e-5)
    y = torch.randn(6, 32, generator=g)
    want = torch.cat([x[:3] + gt[0] * y[:3], x[3:] + gt[1] * y[3:]])
    assert torch.allclose(ref.gate_residual(x.clone(), y, gt, 3), want, atol=1e-6)
    w, b = torch.randn(8, 32, generator=g), torch.randn(8, generator=g)
    assert torch.allclose(ref.linear(x, w, b, gelu=True), F.gelu(F.linear(x, w, b), approximate="tanh"), atol=1e-5)


def test_silu_mul_layouts_and_slabs():
    g = torch.Generator().manual_seed(4)
    gu = torch.randn(3, 16, generator=g)
    assert torch.allclose(ref.silu_mul(gu), F.silu(gu[:, :8]) * gu[:, 8:], atol=1e-6)
    assert torch.allclose(ref.silu_mul(gu, True), F.silu(gu[:, 0::2]) * gu[:, 1::2], atol=1e-6)
    slabs = torch.randn(4, 3, 16, generator=g)
    tot = slabs.sum(0)
    assert torch.allclose(ref.silu_mul(slabs, True).float(), (F.silu(tot[:, 0::2]) * tot[:, 1::2]), atol=2e-2)


def test_qknorm_rope_is_norm_then_rotation():
    g = torch.Generator().manual_seed(5)
    heads, rows = 2, 4
    qkv = torch.randn(rows, 3 * heads * 128, generator=g)
    gq, gk = torch.rand(128, generator=g) + 0.5, torch.rand(128, generator=g) + 0.5
    pos = torch.randint(0, 20, (rows, 2), generator=g, dtype=torch.int32)
    out = ref.qknorm_rope(qkv.clone(), gq, gk, pos, heads)
    q = qkv[:, : heads * 128].view(rows, heads, 128)
    qn = F.rms_norm(q, (128,), gq, 1e-6)
    want = ref.rope(qn, pos, 1e4, 2).reshape(rows, heads * 128)
    assert torch.allclose(out[:, : heads * 128], want, atol=1e-5)
    assert torch.equal(out[:, 2 * heads * 128:], qkv[:, 2 * heads * 128:])   # v untouched
    # a rotation keeps the norm of every (x1, x2) pair
    assert torch.allclose(want.view(rows, heads, 128).norm(dim=-1), qn.norm(dim=-1), atol=1e-4)
