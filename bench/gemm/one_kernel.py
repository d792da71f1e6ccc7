#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Run ONE kernel of the decode step a few times on a small, fixed case: the
target of `ncu` captures (see profiles/).  Weights are larger than L2 or
rotate, launches are few, memory stays within a few GB.

    python bench/gemm/one_kernel.py gate_up|down_slabs|qkv_slabs|lm_head|w8a16|w8a16_int8|attn_decode|rmsnorm|attn_prefill|
                                    attn_joint|attn_joint_small|linear_big|dlin_gate_up|dlin_down|rope_attn [reps]

dlin_gate_up / dlin_down: the decode linears of a TP=8 shard with the collective folded in (gather +
residual + norm prologue and SiLU*mul epilogue; inbox-push epilogue), on the one-rank stand-in for the
link, weights rotating through copies larger than L2.  rope_attn: RoPE + KV write + paged attention +
split merge in one kernel, the TP=8 shard's heads (4 query slots, 1 KV head), batch 64 x 1024 tokens.
"""
import math
import sys
import os

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200.ops import reference as ref  # noqa: E402

which = sys.argv[1] if len(sys.argv) > 1 else "gate_up"
reps = int(sys.argv[2]) if len(sys.argv) > 2 else 3
C = bl.load_extension()
dev = torch.device("cuda", 0)
H, I, B = 3584, 18944, 64
g = torch.Generator(device=dev).manual_seed(0)


def bf(*shape, std=1.0):
    return (torch.randn(*shape, device=dev, generator=g) * std).to(torch.bfloat16)


if which == "gate_up":
    ws = [bf(2 * I, H, std=0.02) for _ in range(2)]
    x = bf(B, H)
    fn = lambda i: C.linear(x, ws[i % 2], None, None, True)  # noqa: E731
elif which == "lm_head":
    w = bf(152064, H, std=0.02)
    x = bf(B, H)
    fn = lambda i: C.linear(x, w)  # noqa: E731
elif which == "down_slabs":
    ws = [bf(H, I, std=0.02) for _ in range(3)]
    x = bf(B, I)
    fn = lambda i: C.linear_partial(x, ws[i % 3])  # noqa: E731
elif which == "qkv_slabs":
    ws = [bf(4608, H, std=0.02) for _ in range(6)]
    x = bf(B, H)
    fn = lambda i: C.linear_partial(x, ws[i % 6])  # noqa: E731
elif which == "w8a16":
    qs = [ref.quantize_w8(torch.randn(2 * I, H, device=dev, generator=g) * 0.02) for _ in range(3)]
    x = bf(B, H)
    fn = lambda i: C.w8a16_linear(x, qs[i % 3][0], qs[i % 3][1])  # noqa: E731
elif which == "w8a16_int8":
    # the same weights, activations quantised per token: k_quant_act + the int8 x int8 GEMM
    qs = [ref.quantize_w8(torch.randn(2 * I, H, device=dev, generator=g) * 0.02) for _ in range(3)]
    x = bf(B, H)
    fn = lambda i: C.w8a16_linear(x, qs[i % 3][0], qs[i % 3][1], act_int8=True)  # noqa: E731
elif which == "attn_decode":
    nq, nkv, hd, bs, ctx = 28, 4, 128, 16, 1024
    nb = B * (ctx // bs)
    kcs = [bf(nb, nkv, bs, hd) for _ in range(2)]
    vcs = [bf(nb, nkv, bs, hd) for _ in range(2)]
    bt = torch.arange(nb, device=dev, dtype=torch.int32).view(B, -1).contiguous()
    cl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
    qkv = bf(B, (nq + 2 * nkv) * hd)
    fn = lambda i: C.paged_attn_decode(qkv, kcs[i % 2], vcs[i % 2], bt, cl, nq, nkv, hd, 1 / math.sqrt(hd), 1)  # noqa: E731
elif which == "rmsnorm":
    x, r, gm = bf(4096, H), bf(4096, H), bf(H)
    fn = lambda i: C.rmsnorm(x, gm, 1e-6, r)  # noqa: E731
elif which == "attn_prefill":
    nq, nkv, hd, S, nb = 28, 4, 128, 1024, 8
    qkv = bf(nb * S, (nq + 2 * nkv) * hd)
    v3 = qkv.view(nb * S, nq + 2 * nkv, hd)
    cu = torch.arange(0, (nb + 1) * S, S, device=dev, dtype=torch.int32)
    fn = lambda i: C.attn_fwd(v3[:, :nq], v3[:, nq:nq + nkv], v3[:, nq + nkv:], cu, cu, S, 1 / math.sqrt(hd), True)  # noqa: E731
elif which in ("attn_joint", "attn_joint_small"):
    # MMDiT joint attention: 24 heads over 4608 tokens (small: 8 heads over 2304)
    nh, hd, L = (24, 128, 4608) if which == "attn_joint" else (8, 128, 2304)
    qkv = bf(L, 3 * nh * hd)
    v3 = qkv.view(L, 3 * nh, hd)
    cu = torch.tensor([0, L], device=dev, dtype=torch.int32)
    fn = lambda i: C.attn_fwd(v3[:, :nh], v3[:, nh:2 * nh], v3[:, 2 * nh:], cu, cu, L, 1 / math.sqrt(hd), False, L)  # noqa: E731
elif which == "linear_big":
    # MMDiT MLP-in at 4608 tokens: [4608, 3072] x [12288, 3072]^T with bias + GELU
    x, w, b = bf(4608, 3072), bf(12288, 3072, std=0.02), bf(12288)
    fn = lambda i: C.linear(x, w, b, None, False, None, gelu=True)  # noqa: E731
elif which in ("dlin_gate_up", "dlin_down"):
    T, inter = B, 2368                      # TP=8 shard of the 7B shape
    link = C.dlin_local_link(T, H, 0)
    res, xn, gamma = bf(T, H), bf(T, H), bf(H)
    wo, a_in = bf(H, 512, std=0.02), bf(T, 512)
    if which == "dlin_gate_up":
        ws = [bf(2 * inter, H, std=0.02) for _ in range(6)]       # 6 x 34 MB

        def fn(i):
            C.dlin(a_in, wo, epi="push", hidden=H, link=link)     # fills the inbox the prologue gathers
            C.dlin(xn, ws[i % 6], pro="gather_norm", epi="silu_mul", residual=res, gamma=gamma, eps=1e-6, link=link)
    else:
        ws = [bf(H, inter, std=0.02) for _ in range(10)]          # 10 x 17 MB
        act = bf(T, inter)

        def fn(i):
            C.dlin(act, ws[i % 10], epi="push", hidden=H, link=link)
            C.gather_norm(xn, res, gamma, 1e-6, link=link)        # consumes the inbox
elif which == "rope_attn":
    nq, nkv, hd, bs, ctx = 4, 1, 128, 16, 1024
    mb = ctx // bs + 2
    nb = B * mb
    kcs = [bf(nb, nkv, bs, hd) for _ in range(4)]
    vcs = [bf(nb, nkv, bs, hd) for _ in range(4)]
    bt = torch.arange(nb, device=dev, dtype=torch.int32).view(B, -1).contiguous()
    cl = torch.full((B,), ctx, device=dev, dtype=torch.int32)
    pos = cl - 1
    slots = (bt[torch.arange(B, device=dev), (pos // bs).long()] * bs + pos % bs).to(torch.int32)
    qkv = bf(B, (nq + 2 * nkv) * hd)
    fn = lambda i: C.rope_attn_decode(qkv, None, pos, slots, kcs[i % 4], vcs[i % 4], bt, cl, nq, nkv, hd, 1e6,  # noqa: E731
                                      1 / math.sqrt(hd), 0)
else:
    raise SystemExit("unknown kernel " + which)

for i in range(2):
    fn(i)
torch.cuda.synchronize()
e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
e0.record()
for i in range(reps):
    fn(i)
e1.record()
torch.cuda.synchronize()
print("%s: %.1f us per launch over %d launches (eager, includes launch gaps)" % (which, e0.elapsed_time(e1) / reps * 1e3, reps))
