# SPDX-License-Identifier: MIT
"""Sharding rules, CPU oracles and package plumbing (no GPU)."""
import pytest
import torch

from barlink_sm86_b200.parallel import head_plan, interleave_gate_up, shard_cols, shard_rows
from barlink_sm86_b200.ops import reference as ref


def test_head_plan_even_split():
    p = head_plan(28, 4, 2, 1)
    assert p.kv_heads == [2, 3] and p.q_heads == list(range(14, 28))
    p = head_plan(28, 4, 4, 3)
    assert p.kv_heads == [3] and p.q_heads == list(range(21, 28))


def test_head_plan_replicates_kv_heads_when_fewer_than_ranks():
    seen = []
    for r in range(8):
        p = head_plan(28, 4, 8, r)
        assert p.nq == 4 and p.nkv == 1 and p.kv_heads == [r // 2]
        for h in p.q_heads:
            if h >= 0:
                assert h // 7 == r // 2  # a query head stays with its KV head
                seen.append(h)
    assert sorted(seen) == list(range(28))  # every head exactly once, the rest are empty slots


def test_head_plan_rejects_impossible_splits():
    with pytest.raises(ValueError):
        head_plan(28, 4, 3, 0)
    with pytest.raises(ValueError):
        head_plan(10, 4, 2, 0)


def test_shards_reassemble():
    w = torch.arange(24.).view(6, 4)
    assert torch.equal(torch.cat([shard_rows(w, 3, r) for r in range(3)], 0), w)
    assert torch.equal(torch.cat([shard_cols(w, 2, r) for r in range(2)], 1), w)
    g, u = torch.zeros(3, 2), torch.ones(3, 2)
    gu = interleave_gate_up(g, u)
    assert torch.equal(gu[0::2], g) and torch.equal(gu[1::2], u)


def test_reference_linear_silu_matches_separate_ops():
    x, g, u = torch.randn(5, 16), torch.randn(8, 16), torch.randn(8, 16)
    got = ref.linear(x, interleave_gate_up(g, u), silu_mul=True)
    want = torch.nn.functional.silu(x @ g.t()) * (x @ u.t())
    assert torch.allclose(got, want, atol=1e-5)


def test_reference_paged_attention_matches_dense():
    torch.manual_seed(0)
    nq, nkv, hd, bs = 4, 2, 16, 16
    ctx = torch.tensor([5, 33])
    kc, vc = torch.randn(6, nkv, bs, hd), torch.randn(6, nkv, bs, hd)
    bt = torch.tensor([[0, 1, 2], [3, 4, 5]], dtype=torch.int32)
    q = torch.randn(2, nq * hd)
    out = ref.paged_attn_decode(q, kc, vc, bt, ctx, nq, nkv, hd, 0.25)
    for b in range(2):
        n = int(ctx[b])
        k = kc[bt[b].long()].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        v = vc[bt[b].long()].permute(1, 0, 2, 3).reshape(nkv, -1, hd)[:, :n]
        qq = q[b].view(nq, 1, hd)
        dense = ref.attention(qq.permute(1, 0, 2), k.permute(1, 0, 2), v.permute(1, 0, 2),
                              [0, 1], [0, n], 0.25, False)
        assert torch.allclose(out[b], dense.reshape(-1), atol=1e-5)


def test_reference_rope_is_a_rotation_and_2d_splits_axes():
    x = torch.randn(7, 3, 32)
    pos = torch.arange(7, dtype=torch.int32)
    y = ref.rope(x, pos, 1e4)
    assert torch.allclose(y.norm(dim=-1), x.norm(dim=-1), atol=1e-4)
    assert torch.allclose(y[0], x[0], atol=1e-6)  # position 0 is the identity
    pos2 = torch.stack([pos, torch.zeros_like(pos)], 1)
    y2 = ref.rope(x, pos2, 1e4, axes=2)
    assert torch.allclose(y2[..., 16:], x[..., 16:], atol=1e-6)  # second axis at position 0


def test_w8_quantisation_round_trip():
    w = torch.randn(32, 64) * 0.02
    wq, s = ref.quantize_w8(w)
    assert wq.dtype == torch.int8 and s.dtype == torch.bfloat16
    back = wq.float() * s.float()[:, None]
    assert (back - w).abs().max() <= s.float().max() * 0.51 + 1e-3


def test_int4_pack_round_trip():
    w = torch.randn(64, 512) * 0.02
    qw, sc, qz = ref.pack_int4(w, 128)
    assert qw.shape == (64, 64) and qw.dtype == torch.int32 and sc.shape == (4, 64) and qz.shape == (4, 8)
    d = ref.w4_dequant(qw, sc, qz, 128)
    step = sc.float().t().repeat_interleave(128, 1)
    assert torch.all((d - w).abs() <= 0.5 * step + 1e-6)
    x = torch.randn(3, 512)
    assert torch.allclose(ref.w4a16_linear(x, qw, sc, qz), x @ d.t(), atol=1e-5)


def test_package_imports_without_a_gpu():
    import barlink_sm86_b200 as bl
    assert callable(bl.init) and callable(bl.allreduce_into) and callable(bl.copy_large)
    import barlink_sm86 as old
    assert old.init is bl.init


def test_mmdit_batches_are_independent_and_sampler_runs():
    """Two samples in one batch give the same rows as each sample alone (joint attention
    must not mix sequences), and the Euler sampler walks the requested number of steps."""
    from barlink_sm86_b200.models import MMDiTConfig, MMDiTModel, MMDiTWeights, denoise, grid_positions
    cfg = MMDiTConfig.tiny()
    m = MMDiTModel(cfg, MMDiTWeights(cfg, "cpu", torch.float32, 3))
    g = torch.Generator().manual_seed(1)
    img = torch.randn(2, 16, cfg.in_channels, generator=g)
    txt = torch.randn(2, 8, cfg.txt_dim, generator=g)
    t = torch.tensor([0.7, 0.2])
    pos = grid_positions(4, 4, "cpu")
    both = m.forward(img, txt, t, pos)
    for b in range(2):
        one = m.forward(img[b:b + 1], txt[b:b + 1], t[b:b + 1], pos)
        assert torch.allclose(both[b:b + 1], one, atol=1e-4, rtol=1e-4)
    calls = []
    orig = m.forward
    m.forward = lambda *a, **k: (calls.append(float(a[2][0])), orig(*a, **k))[1]
    out = denoise(m, img, txt, pos, steps=3)
    assert out.shape == img.shape and torch.isfinite(out).all()
    assert calls == pytest.approx([1.0, 2.0 / 3.0, 1.0 / 3.0])
    assert m.flops_per_forward(1, 4096, 512) > 0


def test_no_comm_control_skips_collectives():
    from barlink_sm86_b200.parallel import TPComm
    c = TPComm.single()
    c.world, c.no_comm = 2, True           # a two-rank communicator whose collectives are switched off
    x = torch.ones(4, 8)
    assert c.all_reduce(x) is x and c.ar_calls == 0
    normed, res = c.allreduce_rmsnorm(x, torch.zeros_like(x), torch.ones(8), 1e-6)
    assert torch.allclose(res, x) and normed.shape == x.shape


def test_w8_group_scales_match_dense_product():
    g = torch.Generator().manual_seed(2)
    w = torch.randn(48, 256, generator=g) * 0.05
    w[:, :128] *= 8.0                       # groups with very different ranges: where group scales matter
    x = torch.randn(5, 256, generator=g)
    wq, sg = ref.quantize_w8_grouped(w, 128)
    assert wq.dtype == torch.int8 and sg.shape == (48, 2)
    yg = ref.w8a16_linear(x, wq, sg)
    wq1, s1 = ref.quantize_w8(w)
    y1 = ref.w8a16_linear(x, wq1, s1)
    want = x @ w.t()
    eg, e1 = (yg - want).norm() / want.norm(), (y1 - want).norm() / want.norm()
    assert eg < 1e-2 and eg < e1            # finer scales, smaller error
    assert torch.allclose(ref.w8_dequant(wq, sg), w, atol=float(sg.float().max()) * 0.51)
