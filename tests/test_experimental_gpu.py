# SPDX-License-Identifier: MIT
"""Kernels that are built but not yet enabled by default.  They run only with
BL_TEST_EXPERIMENTAL=1, against the default path they are meant to replace."""
import math
import os

import pytest
import torch

from conftest import rel_l2

pytestmark = [pytest.mark.gpu,
              pytest.mark.skipif(os.environ.get("BL_TEST_EXPERIMENTAL") != "1",
                                 reason="set BL_TEST_EXPERIMENTAL=1 to run kernels that are not on by default")]


@pytest.mark.parametrize("nq,nkv", [(28, 4), (4, 1), (7, 1), (14, 2)])
@pytest.mark.parametrize("slabs", [0, 3])
@pytest.mark.parametrize("splits", [0, 1, 3])
def test_fused_rope_attention_matches_the_two_kernel_path(ext, nq, nkv, slabs, splits):
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
    got = ext.rope_attn_decode(qkv, bias if slabs else None, pos, slots, k2, v2, bt, ctx, nq, nkv, hd, 1e6, scale,
                               splits)
    assert rel_l2(got, want) < 5e-3
    assert torch.equal(v1, v2)
    assert rel_l2(k2, k1) < 2e-3   # cos/sin come from a shared table here, from sincosf per element there


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


def test_paired_cta_gemm_matches_fp32():
    """The cta_group::2 GEMM (BL_GEMM_PAIR=1, read once per process, hence the child process)."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, BL_GEMM_PAIR="1")
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
