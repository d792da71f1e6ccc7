# SPDX-License-Identifier: MIT
"""Decode linears with the collective folded in (`csrc/dlin_kernels.cu`) on one GPU:
the cluster split-K product against an fp32 statement of the same op, and the
push -> gather + residual + RMSNorm chain through the one-rank stand-in for the link
(the same kernels and inbox protocol that run over NVLink with more ranks)."""
import math

import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _bf(*shape, seed=0, std=1.0):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return (torch.randn(*shape, generator=g, device="cuda") * std).to(torch.bfloat16)


def _rmsnorm(x, gamma, eps):
    xf = x.float()
    y = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)).to(torch.bfloat16).float()
    return (y * gamma.float()).to(torch.bfloat16)


@pytest.mark.parametrize("tokens,n,k,cluster", [
    (64, 768, 3584, 0), (64, 768, 3584, 8), (64, 768, 3584, 5), (64, 3584, 512, 0), (64, 3584, 512, 1),
    (64, 3584, 2368, 4), (7, 300, 512, 3), (1, 256, 128, 0), (16, 1000, 256, 2), (17, 384, 448, 0),
    (33, 512, 4096, 8), (64, 256, 18944, 0), (3, 128, 1376, 7),
])
def test_store_epilogue_matches_fp32(ext, tokens, n, k, cluster):
    x, w = _bf(tokens, k, seed=1), _bf(n, k, seed=2, std=0.05)
    bias = _bf(n, seed=3, std=0.5)
    y = ext.dlin(x, w, epi="store", bias=bias, cluster=cluster)
    torch.cuda.synchronize()
    assert ext.dlin_error_flag(0) == 0
    want = x.float() @ w.float().t() + bias.float()
    assert rel_l2(y, want) < 1e-2, (tokens, n, k, cluster, ext.dlin_cluster(n, k, tokens, cluster))


@pytest.mark.parametrize("tokens,n,k,cluster", [(64, 4736, 3584, 0), (64, 4736, 3584, 4), (5, 512, 256, 2),
                                                (32, 1024, 512, 0)])
def test_silu_mul_epilogue(ext, tokens, n, k, cluster):
    from barlink_sm86_b200.ops import reference as ref
    x, w = _bf(tokens, k, seed=4), _bf(n, k, seed=5, std=0.05)
    y = ext.dlin(x, w, epi="silu_mul", cluster=cluster)
    torch.cuda.synchronize()
    assert ext.dlin_error_flag(0) == 0
    want = ref.linear(x, w, None, None, True)  # interleaved (gate, up) rows
    assert y.shape == (tokens, n // 2)
    assert rel_l2(y, want) < 1e-2


@pytest.mark.parametrize("tokens,hidden,k,n2", [(64, 3584, 512, 768), (8, 1024, 2368, 640), (33, 512, 1376, 256),
                                                (64, 5120, 512, 4736), (5, 8192, 256, 384)])
def test_push_then_gather_norm_chain(ext, tokens, hidden, k, n2):
    """row-parallel linear (push) -> [standalone gather + residual + norm] and
    -> [next linear with the gather in its prologue], several rounds so that the three inbox
    buffers rotate and get cleared, against the unfused statement."""
    eps = 1e-6
    link = ext.dlin_local_link(tokens, hidden, 0)
    gamma = (1.0 + _bf(hidden, seed=6, std=0.1).float()).to(torch.bfloat16)
    w1 = _bf(hidden, k, seed=7, std=0.05)
    w2 = _bf(n2, hidden, seed=8, std=0.05)
    res = _bf(tokens, hidden, seed=9)
    res_ref = res.clone()
    xn = torch.empty(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    for it in range(7):
        a = _bf(tokens, k, seed=20 + it)
        ext.dlin(a, w1, epi="push", hidden=hidden, link=link, cluster=(it % 3) + 1)
        part = (a.float() @ w1.float().t()).to(torch.bfloat16)
        res_ref = (part.float() + res_ref.float()).to(torch.bfloat16)
        want_xn = _rmsnorm(res_ref, gamma, eps)
        if it % 2 == 0:
            ext.gather_norm(xn, res, gamma, eps, link=link)
            torch.cuda.synchronize()
            assert rel_l2(xn, want_xn) < 6e-3, it
        else:
            # in-kernel form: the operand buffer receives residual * gamma, the 1 / rms of each
            # token is applied to the product by the epilogue
            bias = _bf(n2, seed=40 + it, std=0.3)
            y = ext.dlin(xn, w2, pro="gather_norm", epi="store", bias=bias, residual=res, gamma=gamma, eps=eps,
                         link=link, cluster=(it % 4) + 1)
            torch.cuda.synchronize()
            want_y = want_xn.float() @ w2.float().t() + bias.float()
            assert rel_l2(y, want_y) < 1.5e-2, it
            assert rel_l2(xn, (res_ref.float() * gamma.float()).to(torch.bfloat16)) < 6e-3, it
        assert ext.dlin_error_flag(0) == 0, it
        assert rel_l2(res, res_ref) < 4e-3, it


def test_chain_inside_a_cuda_graph(ext):
    """The chain is replay-safe: expectations are device counters, nothing is baked in at capture."""
    tokens, hidden, k, n2, eps = 16, 1024, 512, 384, 1e-6
    link = ext.dlin_local_link(tokens, hidden, 0)
    gamma = torch.ones(hidden, dtype=torch.bfloat16, device="cuda")
    w1, w2 = _bf(hidden, k, seed=1, std=0.05), _bf(n2, hidden, seed=2, std=0.05)
    a = _bf(tokens, k, seed=3)
    res = torch.zeros(tokens, hidden, dtype=torch.bfloat16, device="cuda")
    xn = torch.empty_like(res)
    y = torch.empty(tokens, n2, dtype=torch.bfloat16, device="cuda")

    def body():
        ext.dlin(a, w1, epi="push", hidden=hidden, link=link)
        ext.dlin(xn, w2, pro="gather_norm", epi="store", out=y, residual=res, gamma=gamma, eps=eps, link=link)

    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        body()
    torch.cuda.current_stream().wait_stream(s)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        body()
    res.zero_()
    part = (a.float() @ w1.float().t()).to(torch.bfloat16)
    ref = torch.zeros_like(res)
    for it in range(5):
        g.replay()
        torch.cuda.synchronize()
        ref = (part.float() + ref.float()).to(torch.bfloat16)
        assert ext.dlin_error_flag(0) == 0
        assert rel_l2(res, ref) < 4e-3, it
        assert rel_l2(y, _rmsnorm(ref, gamma, eps).float() @ w2.float().t()) < 1.5e-2, it


@pytest.mark.parametrize("nq,nkv", [(28, 4), (4, 1), (7, 1), (14, 2)])
@pytest.mark.parametrize("slabs", [0, 3])
@pytest.mark.parametrize("splits,merge", [(0, True), (1, True), (3, True), (3, False), (5, True)])
def test_fused_rope_attention_matches_the_two_kernel_path(ext, nq, nkv, slabs, splits, merge):
    """RoPE + KV write + paged attention in one launch against rope_kv_write followed by
    paged_attn_decode: same attention output, same cache contents."""
    hd, bs = 128, 16
    ctxs = [1, 16, 17, 300, 1024, 33, 640, 5]
    batch, max_blocks = len(ctxs), 64
    g = torch.Generator(device="cuda").manual_seed(nq * 10 + slabs)
    width = (nq + 2 * nkv) * hd
    nblk = batch * max_blocks
    kc = (torch.randn(nblk, nkv, bs, hd, device="cuda", generator=g) * 0.5).bfloat16()
    vc = (torch.randn(nblk, nkv, bs, hd, device="cuda", generator=g) * 0.5).bfloat16()
    bt = torch.randperm(nblk, device="cuda", generator=g).to(torch.int32).view(batch, max_blocks).contiguous()
    ctx = torch.tensor(ctxs, dtype=torch.int32, device="cuda")
    pos = ctx - 1
    slots = (bt[torch.arange(batch, device="cuda"), (pos // bs).long()] * bs + pos % bs).to(torch.int32)
    bias = (torch.randn(width, device="cuda", generator=g) * 0.1).bfloat16()
    if slabs:
        qkv = torch.randn(slabs, batch, width, device="cuda", generator=g) * 0.3
    else:
        qkv = (torch.randn(batch, width, device="cuda", generator=g) * 0.5).bfloat16()
    scale = 1.0 / math.sqrt(hd)
    k1, v1, k2, v2 = kc.clone(), vc.clone(), kc.clone(), vc.clone()
    rot = ext.rope_kv_write(qkv.clone(), pos, slots, k1, v1, nq, nkv, hd, bs, 1e6, bias if slabs else None)
    want = ext.paged_attn_decode(rot, k1, v1, bt, ctx, nq, nkv, hd, scale, splits)
    for _ in range(2):  # twice: the in-kernel merge must leave its counters at zero
        k2.copy_(kc)
        v2.copy_(vc)
        got = ext.rope_attn_decode(qkv, bias if slabs else None, pos, slots, k2, v2, bt, ctx, nq, nkv, hd, 1e6,
                                   scale, splits, merge)
    assert rel_l2(got, want) < 5e-3
    assert torch.equal(v1, v2)
    assert rel_l2(k2, k1) < 2e-3   # cos/sin come from a shared table here, from sincosf per element there
