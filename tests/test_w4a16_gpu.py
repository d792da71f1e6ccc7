# SPDX-License-Identifier: MIT
"""Int4 weight-only linear (GPTQ-v1 tensors) against the fp32 statement: the
decode GEMV for 1..16 rows, every k-split, and the widen + GEMM path."""
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu

# (K, N) of the reference's int4 MLP shapes (demos/qwen_tp/int4linear.py:152) plus small odd ones
SHAPES = [(5120, 17408), (17408, 5120), (5120, 6144), (256, 64), (1024, 8 * 37)]


@pytest.mark.parametrize("k,n", SHAPES)
@pytest.mark.parametrize("m", [1, 2, 3, 8, 16])
def test_w4a16_gemv(ext, k, n, m):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(k + m)
    w = torch.randn(n, k, generator=g) * 0.02
    x = torch.randn(m, k, generator=g).bfloat16()
    qw, sc, qz = ops.ref.pack_int4(w)
    want = ops.ref.w4a16_linear(x, qw, sc, qz)
    got = ops.w4a16_linear(x.cuda(), qw.cuda(), sc.cuda(), qz.cuda()).cpu()
    assert rel_l2(got, want) < 5e-3


@pytest.mark.parametrize("splits", [1, 2, 5, 40])
def test_w4a16_gemv_splits_and_groups(ext, splits):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(splits)
    k, n, group = 2048, 512, 64
    w = torch.randn(n, k, generator=g) * 0.05
    x = torch.randn(4, k, generator=g).bfloat16()
    qw, sc, qz = ops.ref.pack_int4(w, group)
    # zero points other than 8: the kernel must read them per output
    z = torch.randint(5, 12, (k // group, n), generator=g)
    qz = sum(z.view(k // group, n // 8, 8)[..., j].long() << (4 * j) for j in range(8))
    qz = ((qz + 2 ** 31) % 2 ** 32 - 2 ** 31).to(torch.int32)
    want = ops.ref.w4a16_linear(x, qw, sc, qz, group)
    a = ext.w4a16_linear(x.cuda(), qw.cuda(), sc.cuda(), qz.cuda(), group, splits)
    b = ext.w4a16_linear(x.cuda(), qw.cuda(), sc.cuda(), qz.cuda(), group, splits)
    assert rel_l2(a.cpu(), want) < 5e-3
    assert torch.equal(a, b)  # fixed reduction order: bit-identical run to run


def test_w4a16_prefill_path_and_dequant(ext):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(9)
    k, n = 1024, 768
    w = torch.randn(n, k, generator=g) * 0.02
    qw, sc, qz = ops.ref.pack_int4(w)
    dq = ext.w4_dequant(qw.cuda(), sc.cuda(), qz.cuda(), 128).float().cpu()
    assert rel_l2(dq, ops.ref.w4_dequant(qw, sc, qz)) < 5e-3
    x = torch.randn(100, k, generator=g).bfloat16()
    got = ops.w4a16_linear(x.cuda(), qw.cuda(), sc.cuda(), qz.cuda()).cpu()
    assert rel_l2(got, ops.ref.w4a16_linear(x, qw, sc, qz)) < 1e-2
