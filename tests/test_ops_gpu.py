# SPDX-License-Identifier: MIT
"""Numerics of the single-GPU sm_100a kernels against fp32 PyTorch statements
of the same ops (`barlink_sm86_b200.ops.reference`)."""
import math

import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * std).to(torch.bfloat16)


@pytest.mark.parametrize("tokens,n,k", [
    (1, 256, 128), (7, 384, 448), (16, 1000, 256), (33, 512, 4096), (64, 3584, 1024),
    (128, 640, 192), (64, 256, 18944),
])
def test_linear_decode_orientation(ext, tokens, n, k):
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(tokens, k, seed=1), _bf(n, k, seed=2, std=0.05)
    y = ext.linear(x, w)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    want = ref.linear(x, w)
    assert rel_l2(y, want) < 1e-2, (tokens, n, k)


@pytest.mark.parametrize("tokens,n,k", [(256, 512, 256), (300, 640, 320), (1024, 1024, 512), (130, 264, 64)])
def test_linear_prefill_orientation(ext, tokens, n, k):
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(tokens, k, seed=3), _bf(n, k, seed=4, std=0.05)
    y = ext.linear(x, w)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    assert rel_l2(y, ref.linear(x, w)) < 1e-2


@pytest.mark.parametrize("bn", [16, 32, 64, 128, 256])
@pytest.mark.parametrize("swap", [0, 1])
def test_linear_every_tile_width(ext, bn, swap):
    from barlink_sm86_b200.ops import reference as ref
    tokens, n, k = (48, 384, 512) if swap else (384, 520, 512)
    x, w = _bf(tokens, k, seed=5), _bf(n, k, seed=6, std=0.05)
    y = ext.linear(x, w, force_swap=swap, bn=bn)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    assert rel_l2(y, ref.linear(x, w)) < 1e-2


@pytest.mark.parametrize("splits", [1, 2, 5, 8])
def test_linear_split_k_is_deterministic(ext, splits):
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(24, 2048, seed=7), _bf(256, 2048, seed=8, std=0.05)
    y1 = ext.linear(x, w, splits=splits)
    y2 = ext.linear(x, w, splits=splits)
    torch.cuda.synchronize()
    assert torch.equal(y1, y2)
    assert rel_l2(y1, ref.linear(x, w)) < 1e-2


@pytest.mark.parametrize("tokens", [5, 64, 200])
def test_linear_epilogues(ext, tokens):
    from barlink_sm86_b200.ops import reference as ref
    n, k = 512, 256
    x, w = _bf(tokens, k, seed=9), _bf(n, k, seed=10, std=0.05)
    b, r = _bf(n, seed=11), _bf(tokens, n, seed=12)
    assert rel_l2(ext.linear(x, w, b), ref.linear(x, w, b)) < 1e-2
    assert rel_l2(ext.linear(x, w, b, r), ref.linear(x, w, b, r)) < 1e-2
    got = ext.linear(x, w, None, None, True)
    want = ref.linear(x, w, silu_mul=True)
    assert got.shape == (tokens, n // 2)
    assert rel_l2(got, want) < 2e-2
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0


@pytest.mark.parametrize("rows,hidden", [(1, 3584), (64, 3584), (3, 5120), (17, 512), (5, 8192)])
def test_rmsnorm(ext, rows, hidden):
    from barlink_sm86_b200.ops import reference as ref
    x, g = _bf(rows, hidden, seed=1), _bf(hidden, seed=2)
    out, _ = ext.rmsnorm(x, g, 1e-6)
    want, _ = ref.rmsnorm(x, g, 1e-6)
    assert rel_l2(out, want) < 5e-3
    res = _bf(rows, hidden, seed=3)
    res_c = res.clone()
    out, new_res = ext.rmsnorm(x, g, 1e-6, res)
    want, want_res = ref.rmsnorm(x, g, 1e-6, res_c)
    assert torch.equal(new_res, want_res)
    assert rel_l2(out, want) < 5e-3


def test_rope_kv_write(ext):
    from barlink_sm86_b200.ops import reference as ref
    rows, nq, nkv, hd, bs = 9, 7, 2, 128, 16
    qkv = _bf(rows, (nq + 2 * nkv) * hd, seed=1)
    pos = torch.tensor([0, 1, 5, 17, 100, 1023, 31, 32, 4000], dtype=torch.int32, device="cuda")
    slots = torch.tensor([3, 17, 40, -1, 64, 65, 2, 99, 130], dtype=torch.int32, device="cuda")
    kc = torch.zeros(10, nkv, bs, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    q2, kc2, vc2 = qkv.clone(), kc.clone(), vc.clone()
    ext.rope_kv_write(qkv, pos, slots, kc, vc, nq, nkv, hd, bs, 1e6)
    ref.rope_kv_write(q2, pos, slots, kc2, vc2, nq, nkv, hd, bs, 1e6)
    assert rel_l2(qkv, q2) < 5e-3
    assert rel_l2(kc, kc2) < 5e-3
    assert torch.equal(vc, vc2)


def test_rope_2d(ext):
    from barlink_sm86_b200.ops import reference as ref
    rows, heads, hd = 33, 3, 128
    x = _bf(rows, heads, hd, seed=4)
    pos = torch.randint(0, 64, (rows, 2), dtype=torch.int32, device="cuda")
    want = ref.rope(x.clone(), pos, 1e4, axes=2)
    ext.rope(x.view(rows, heads * hd), pos.contiguous(), heads, hd, 1e4, 2)
    assert rel_l2(x, want) < 5e-3


@pytest.mark.parametrize("interleaved", [False, True])
def test_silu_mul(ext, interleaved):
    from barlink_sm86_b200.ops import reference as ref
    gu = _bf(13, 2 * 1376, seed=5)
    assert rel_l2(ext.silu_mul(gu, interleaved), ref.silu_mul(gu, interleaved)) < 5e-3


def test_embedding_and_argmax(ext):
    from barlink_sm86_b200.ops import reference as ref
    table = _bf(1000, 512, seed=6)
    ids = torch.tensor([0, 5, 999, 1000, 250], dtype=torch.int32, device="cuda")
    assert torch.equal(ext.embedding(ids, table, 0), ref.embedding(ids, table, 0))
    assert torch.equal(ext.embedding(ids, table[200:600].contiguous(), 200),
                       ref.embedding(ids, table[200:600], 200))
    logits = _bf(9, 152064, seed=7)
    logits[3, 77] = 100.0
    logits[4, 5] = logits[4, 4000] = 50.0  # tie: lowest index wins
    idx, val = ext.argmax(logits, 10)
    want_idx, want_val = ref.argmax(logits, 10)
    assert torch.equal(idx, want_idx)
    assert torch.equal(val, want_val)
    assert idx[4].item() == 15


@pytest.mark.parametrize("nq,nkv", [(28, 4), (4, 1), (14, 2), (16, 1)])
@pytest.mark.parametrize("splits", [1, 0, 3])
def test_paged_attention_decode(ext, nq, nkv, splits):
    from barlink_sm86_b200.ops import reference as ref
    batch, hd, bs, max_blocks = 5, 128, 16, 40
    ctx = torch.tensor([1, 16, 17, 300, 640], dtype=torch.int32, device="cuda")
    n_blocks = batch * max_blocks
    kc = _bf(n_blocks, nkv, bs, hd, seed=1)
    vc = _bf(n_blocks, nkv, bs, hd, seed=2)
    perm = torch.randperm(n_blocks, device="cuda", generator=torch.Generator("cuda").manual_seed(3))
    bt = perm.to(torch.int32).view(batch, max_blocks).contiguous()
    qkv = _bf(batch, (nq + 2 * nkv) * hd, seed=4)
    scale = 1.0 / math.sqrt(hd)
    got = ext.paged_attn_decode(qkv, kc, vc, bt, ctx, nq, nkv, hd, scale, splits)
    want = ref.paged_attn_decode(qkv, kc, vc, bt, ctx, nq, nkv, hd, scale)
    assert rel_l2(got, want) < 1e-2


@pytest.mark.parametrize("tokens,n,k,splits", [(64, 4608, 3584, 4), (8, 3584, 18944, 5), (1, 512, 1024, 2),
                                               (33, 640, 1024, 3)])
def test_linear_split_slabs_sum_to_the_product(ext, tokens, n, k, splits):
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(tokens, k, seed=21), _bf(n, k, seed=22, std=0.05)
    slabs = ext.linear_partial(x, w, splits)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    assert slabs.shape == (splits, tokens, n) and slabs.dtype == torch.float32
    want = x.float() @ w.float().t()
    assert rel_l2(slabs.sum(0), want) < 1e-3


def test_rmsnorm_and_rope_consume_slabs(ext):
    from barlink_sm86_b200.ops import reference as ref
    rows, hidden, S = 9, 3584, 4
    g = torch.Generator(device="cuda").manual_seed(5)
    slabs = torch.randn(S, rows, hidden, device="cuda", generator=g)
    gamma, res = _bf(hidden, seed=6), _bf(rows, hidden, seed=7)
    x = slabs.sum(0).to(torch.bfloat16)
    want, want_res = ref.rmsnorm(x, gamma, 1e-6, res.clone())
    got, got_res = ext.rmsnorm(slabs, gamma, 1e-6, res)
    assert torch.equal(got_res, want_res)
    assert rel_l2(got, want) < 5e-3
    # rope + kv write from slabs with bias
    nq, nkv, hd, bs = 7, 2, 128, 16
    width = (nq + 2 * nkv) * hd
    slabs = torch.randn(3, rows, width, device="cuda", generator=g)
    bias = _bf(width, seed=8)
    pos = torch.arange(rows, dtype=torch.int32, device="cuda") * 37
    slots = torch.arange(rows, dtype=torch.int32, device="cuda") * 3 + 1
    kc = torch.zeros(4, nkv, bs, hd, dtype=torch.bfloat16, device="cuda")
    vc = torch.zeros_like(kc)
    kc2, vc2 = kc.clone(), vc.clone()
    q_in = (slabs.sum(0) + bias.float()).to(torch.bfloat16)
    want = ref.rope_kv_write(q_in.clone(), pos, slots, kc2, vc2, nq, nkv, hd, bs, 1e6)
    got = ext.rope_kv_write(slabs, pos, slots, kc, vc, nq, nkv, hd, bs, 1e6, bias)
    assert rel_l2(got, want) < 5e-3
    assert rel_l2(kc, kc2) < 5e-3
    assert torch.equal(vc, vc2)


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("nq,nkv", [(4, 1), (6, 2)])
def test_dense_attention(ext, causal, nq, nkv):
    from barlink_sm86_b200.ops import reference as ref
    hd = 128
    lens_q = [70, 1, 129, 64]
    lens_k = lens_q if causal else [70, 33, 200, 64]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = _bf(sum(lens_q), nq, hd, seed=1)
    k = _bf(sum(lens_k), nkv, hd, seed=2)
    v = _bf(sum(lens_k), nkv, hd, seed=3)
    scale = 1.0 / math.sqrt(hd)
    got = ext.attn_fwd(q, k, v, cu_q, cu_k, max(lens_q), scale, causal)
    want = ref.attention(q, k, v, cu_q.cpu(), cu_k.cpu(), scale, causal)
    assert rel_l2(got, want) < 1e-2


def test_dense_attention_on_fused_qkv_views(ext):
    from barlink_sm86_b200.ops import reference as ref
    T, nq, nkv, hd = 200, 4, 1, 128
    qkv = _bf(T, (nq + 2 * nkv) * hd, seed=4)
    v3 = qkv.view(T, nq + 2 * nkv, hd)
    cu = torch.tensor([0, 120, 200], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    got = ext.attn_fwd(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu, cu, 120, scale, True)
    want = ref.attention(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu.cpu(), cu.cpu(), scale, True)
    assert rel_l2(got, want) < 1e-2


@pytest.mark.parametrize("splits,rows,inter", [(4, 64, 2368), (2, 7, 4736), (1, 128, 64)])
def test_silu_mul_over_k_split_slabs(ext, splits, rows, inter):
    from barlink_sm86_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(inter)
    slabs = torch.randn(splits, rows, 2 * inter, device="cuda", generator=g)
    got = ext.silu_mul(slabs, True)
    want = ref.silu_mul(slabs, True)
    assert got.dtype == torch.bfloat16 and rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("causal", [True, False])
@pytest.mark.parametrize("nq,nkv", [(4, 1), (6, 2), (3, 3)])
def test_dense_attention_tensor_core(ext, causal, nq, nkv):
    """The tcgen05 kernel (selected by max_k) against the fp32 statement:
    ragged packed sequences, tiles with one or both 128-row halves in use, key
    counts off the 64-key step, scores large enough to force a rescale."""
    from barlink_sm86_b200.ops import reference as ref
    hd = 128
    lens_q = [70, 1, 129, 64, 300, 513]
    lens_k = lens_q if causal else [70, 33, 200, 64, 1000, 257]
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = _bf(sum(lens_q), nq, hd, seed=1) * 3
    k = _bf(sum(lens_k), nkv, hd, seed=2) * 3
    v = _bf(sum(lens_k), nkv, hd, seed=3)
    scale = 1.0 / math.sqrt(hd)
    got = ext.attn_fwd(q, k, v, cu_q, cu_k, max(lens_q), scale, causal, max(lens_k))
    want = ref.attention(q, k, v, cu_q.cpu(), cu_k.cpu(), scale, causal)
    assert ext.attn_error_flag(0) == 0
    assert rel_l2(got, want) < 1e-2


def test_dense_attention_tensor_core_on_fused_qkv_views(ext):
    from barlink_sm86_b200.ops import reference as ref
    T, nq, nkv, hd = 1200, 4, 4, 128
    qkv = _bf(T, (nq + 2 * nkv) * hd + 256, seed=4)
    v3 = qkv[:, : (nq + 2 * nkv) * hd].unflatten(1, (nq + 2 * nkv, hd))
    cu = torch.tensor([0, 600, 1200], dtype=torch.int32, device="cuda")
    scale = 1.0 / math.sqrt(hd)
    got = ext.attn_fwd(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu, cu, 600, scale, False, 600)
    want = ref.attention(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu.cpu(), cu.cpu(), scale, False)
    assert ext.attn_error_flag(0) == 0
    assert rel_l2(got, want) < 1e-2


@pytest.mark.parametrize("tokens,n,k", [(64, 4608, 3584), (7, 1000, 448), (300, 640, 320), (1024, 1024, 512),
                                        (16, 256, 18944), (200, 300, 200)])
def test_linear_with_pretiled_weights(ext, tokens, n, k):
    """Weights stored as swizzled 16 KiB tiles (one bulk copy per tile) give the
    same result as the row-major weight, in both orientations and with k-splits."""
    from barlink_sm86_b200 import ops
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(tokens, k, seed=31), _bf(n, k, seed=32, std=0.05)
    tw = ops.tile_weight(w)
    assert isinstance(tw, ops.TiledWeight) and tw.shape == (n, k)
    assert torch.equal(ops.untile_weight(tw), w)
    got = ops.linear(x, tw)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    assert rel_l2(got, ref.linear(x, w)) < 1e-2
    if tokens < 512:
        assert torch.equal(got, ext.linear(x, w))  # same arithmetic, different fetch
    else:
        assert rel_l2(got, ext.linear(x, w)) < 1e-3  # the row-major weight takes the paired-CTA kernel here
    if tokens <= 128:
        slabs = ops.linear_split(x, tw)
        total = slabs.sum(0) if slabs.dtype == torch.float32 else slabs.float()
        assert rel_l2(total, x.float() @ w.float().t()) < 1e-2


PAIR_SCRIPT = r"""
import os, sys, torch
sys.path.insert(0, %r)
from barlink_sm86_b200 import ops, load_extension
C = load_extension()
g = torch.Generator(device="cuda").manual_seed(0)
worst = 0.0
for m, n, k, extra in [(4608, 3072, 3072, "bias"), (1000, 300, 512, "none"), (512, 256, 64, "gelu"),
                       (2304, 9216, 3072, "gelu"), (777, 1024, 1536, "residual"), (4608, 3072, 12288, "bias")]:
    x = (torch.randn(m, k, device="cuda", generator=g) * 0.5).bfloat16()
    w = (torch.randn(n, k, device="cuda", generator=g) / k ** 0.5).bfloat16()
    b = torch.randn(n, device="cuda", generator=g).bfloat16()
    res = torch.randn(m, n, device="cuda", generator=g).bfloat16() if extra == "residual" else None
    y = ops.linear(x, w, None if extra == "none" else b, residual=res, gelu=extra == "gelu")
    want = ops.ref.linear(x, w, None if extra == "none" else b, residual=res, gelu=extra == "gelu").float()
    err = ((y.float() - want).norm() / want.norm()).item()
    worst = max(worst, err)
    assert err < 1e-2, (m, n, k, extra, err)
torch.cuda.synchronize()
assert C.gemm_error_flag(0) == 0
print("PAIR OK worst rel-L2 %%.4f" %% worst)
"""


@pytest.mark.parametrize("pair", ["1", "0"])
def test_large_token_major_gemm_paired_and_single_cta(pair):
    """Token-major products of 512 tokens or more: the cta_group::2 kernel (default) and the
    single-CTA kernel (BL_GEMM_PAIR=0; the switch is read once per process, hence the child)."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, BL_GEMM_PAIR=pair)
    p = subprocess.run([sys.executable, "-c", PAIR_SCRIPT % root], capture_output=True, text=True, timeout=120, env=env)
    assert p.returncode == 0 and "PAIR OK" in p.stdout, p.stdout[-1500:] + p.stderr[-3000:]


@pytest.mark.parametrize("nq,nkv", [(4, 1), (3, 3)])
def test_tensor_core_attention_causal_with_longer_keys(ext, nq, nkv):
    """Causal attention where the keys start before the queries (a later chunk of a chunked
    prefill): the last query sees the last key, both kernels against the fp32 statement."""
    from barlink_sm86_b200.ops import reference as ref
    hd = 128
    lens_q = [70, 1, 129, 300]
    lens_k = [200, 64, 129, 813]
    g = torch.Generator(device="cuda").manual_seed(nq)
    cu_q = torch.tensor([0] + list(torch.tensor(lens_q).cumsum(0)), dtype=torch.int32, device="cuda")
    cu_k = torch.tensor([0] + list(torch.tensor(lens_k).cumsum(0)), dtype=torch.int32, device="cuda")
    q = torch.randn(sum(lens_q), nq, hd, device="cuda", generator=g).bfloat16()
    k = torch.randn(sum(lens_k), nkv, hd, device="cuda", generator=g).bfloat16()
    v = torch.randn(sum(lens_k), nkv, hd, device="cuda", generator=g).bfloat16()
    scale = 1.0 / math.sqrt(hd)
    want = ref.attention(q, k, v, cu_q.cpu(), cu_k.cpu(), scale, True)
    got_tc = ext.attn_fwd(q, k, v, cu_q, cu_k, max(lens_q), scale, True, max(lens_k))
    got_mma = ext.attn_fwd(q, k, v, cu_q, cu_k, max(lens_q), scale, True)
    assert ext.attn_error_flag(0) == 0
    assert rel_l2(got_tc, want) < 1e-2
    assert rel_l2(got_mma, want) < 1e-2
