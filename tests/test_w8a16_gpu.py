# SPDX-License-Identifier: MIT
"""W8A16: the tcgen05 kernel that widens int8 weights in its main loop, and the
reference-compatible quant_act/gemm pair, against fp64 statements on the
quantised operands (the reference's criterion: rel-L2 < 2e-2,
torch_ext/tests/test_w8a16.py:45-49 there)."""
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu


def _quant(n, k, seed):
    from barlink_sm86_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(seed)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    return ref.quantize_w8(w)


@pytest.mark.parametrize("m,n,k", [(1, 512, 3072), (3, 5120, 5120), (16, 1024, 8704), (64, 27648 // 8 * 2, 5120),
                                   (64, 5120, 3456), (200, 640, 512)])
def test_w8a16_linear(ext, m, n, k):
    from barlink_sm86_b200.ops import reference as ref
    wq, scale = _quant(n, k, 1)
    x = torch.randn(m, k, device="cuda", generator=torch.Generator("cuda").manual_seed(2)).to(torch.bfloat16)
    got = ext.w8a16_linear(x, wq, scale)
    torch.cuda.synchronize()
    assert ext.w8_error_flag(0) == 0
    want = (x.double() @ wq.double().t()) * scale.double()[None, :]
    assert rel_l2(got, want) < 1e-2, (m, n, k)
    assert rel_l2(got, ref.w8a16_linear(x, wq, scale)) < 1e-2


@pytest.mark.parametrize("m,n,k", [(1, 512, 3072), (3, 5120, 5120), (16, 1024, 8704), (64, 27648 // 8 * 2, 5120),
                                   (64, 5120, 3456), (33, 640, 80), (200, 640, 512), (600, 768, 1024)])
def test_w8a16_linear_with_int8_activations(ext, m, n, k):
    """Activations quantised per token, int8 x int8 on the tensor cores (tcgen05.mma kind::i8): equal to
    the integer arithmetic of the fp32 statement up to the bf16 rounding of the output, and within the
    reference's tolerance of the unquantised product."""
    from barlink_sm86_b200.ops import reference as ref
    wq, scale = _quant(n, k, 11)
    x = torch.randn(m, k, device="cuda", generator=torch.Generator("cuda").manual_seed(12)).to(torch.bfloat16)
    got = ext.w8a16_linear(x, wq, scale, act_int8=True)
    torch.cuda.synchronize()
    assert ext.w8_error_flag(0) == 0 and ext.gemm_error_flag(0) == 0
    assert rel_l2(got, ref.w8a8_dynamic_linear(x, wq, scale)) < 5e-3, (m, n, k)
    want = (x.double() @ wq.double().t()) * scale.double()[None, :]
    assert rel_l2(got, want) < 2e-2, (m, n, k)
    x[0, 5] = 9.0   # an outlier sets the token's scale: coarser steps, the same integer arithmetic
    got = ext.w8a16_linear(x, wq, scale, act_int8=True)
    assert rel_l2(got, ref.w8a8_dynamic_linear(x, wq, scale)) < 5e-3, (m, n, k)


@pytest.mark.parametrize("m,n,k,group", [(1, 512, 3072, 128), (5, 5120, 5120, 128), (16, 1024, 8704, 128),
                                         (64, 6912, 5120, 128), (33, 640, 1024, 256), (64, 300, 384, 128)])
def test_w8a16_int8_activations_with_group_scales(ext, m, n, k, group):
    """Group-128 weight scales (the reference's checkpoint format) with int8 activations: every k-block of
    128 is multiplied into an accumulator of its own and the epilogue warps add acc * scale[row][group]."""
    from barlink_sm86_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(21)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    w[:, : k // 2] *= 4.0   # groups of different magnitude: the scales matter
    wq, scale = ref.quantize_w8_grouped(w, group)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda", generator=g).to(torch.bfloat16)
    got = ext.w8a16_linear(x, wq, scale, bias, act_int8=True, group_scale=scale)
    torch.cuda.synchronize()
    assert ext.gemm_error_flag(0) == 0
    assert rel_l2(got, ref.w8a8_dynamic_linear(x, wq, scale, bias)) < 5e-3, (m, n, k)
    want = x.double() @ ref.w8_dequant(wq, scale).double().t() + bias.double()
    assert rel_l2(got, want) < 2e-2, (m, n, k)
    if n % 2 == 0:
        got = ext.w8a16_linear(x, wq, scale, None, True, act_int8=True, group_scale=scale)
        assert rel_l2(got, ref.w8a8_dynamic_linear(x, wq, scale, None, True)) < 1e-2
    again = ext.w8a16_linear(x, wq, scale, bias, act_int8=True, group_scale=scale)
    assert torch.equal(again, ext.w8a16_linear(x, wq, scale, bias, act_int8=True, group_scale=scale))


def test_w8a16_int8_activations_epilogues_splits_and_row_pitch(ext):
    from barlink_sm86_b200.ops import reference as ref
    m, n, k = 8, 1024, 4096
    wq, scale = _quant(n, k, 13)
    wide = torch.randn(m, k + 64, device="cuda", generator=torch.Generator("cuda").manual_seed(14)).to(torch.bfloat16)
    x = wide[:, :k]   # row pitch larger than k
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    assert rel_l2(ext.w8a16_linear(x, wq, scale, bias, act_int8=True), ref.w8a8_dynamic_linear(x, wq, scale, bias)) < 5e-3
    assert rel_l2(ext.w8a16_linear(x, wq, scale, None, True, act_int8=True),
                  ref.w8a8_dynamic_linear(x, wq, scale, None, True)) < 1e-2
    a = ext.w8a16_linear(x, wq, scale, None, False, 4, act_int8=True)
    b = ext.w8a16_linear(x, wq, scale, None, False, 4, act_int8=True)
    assert torch.equal(a, b)
    assert rel_l2(a, ref.w8a8_dynamic_linear(x, wq, scale)) < 5e-3
    # prefill orientation with the SiLU*mul epilogue
    xp = torch.randn(700, k, device="cuda", generator=torch.Generator("cuda").manual_seed(15)).to(torch.bfloat16)
    assert rel_l2(ext.w8a16_linear(xp, wq, scale, bias, True, act_int8=True),
                  ref.w8a8_dynamic_linear(xp, wq, scale, bias, True)) < 1e-2


def test_w8a16_linear_epilogues_and_splits(ext):
    from barlink_sm86_b200.ops import reference as ref
    m, n, k = 8, 1024, 4096
    wq, scale = _quant(n, k, 3)
    x = torch.randn(m, k, device="cuda", generator=torch.Generator("cuda").manual_seed(4)).to(torch.bfloat16)
    bias = torch.randn(n, device="cuda").to(torch.bfloat16)
    assert rel_l2(ext.w8a16_linear(x, wq, scale, bias), ref.w8a16_linear(x, wq, scale, bias)) < 1e-2
    assert rel_l2(ext.w8a16_linear(x, wq, scale, None, True), ref.w8a16_linear(x, wq, scale, None, True)) < 2e-2
    a = ext.w8a16_linear(x, wq, scale, None, False, 4)
    b = ext.w8a16_linear(x, wq, scale, None, False, 4)
    assert torch.equal(a, b)
    assert rel_l2(a, ref.w8a16_linear(x, wq, scale)) < 1e-2


def test_w8a16_prefill_path(ext):
    from barlink_sm86_b200.ops import reference as ref
    wq, scale = _quant(768, 1024, 5)
    x = torch.randn(600, 1024, device="cuda").to(torch.bfloat16)
    assert rel_l2(ext.w8a16_linear(x, wq, scale), ref.w8a16_linear(x, wq, scale)) < 1.5e-2


@pytest.mark.parametrize("M", [1, 3, 16])
@pytest.mark.parametrize("S", [1, 4, 7])
def test_reference_api_pair(ext, M, S):
    N, K = 1536, 3072
    g = torch.Generator(device="cuda").manual_seed(6)
    wq = torch.randint(-127, 128, (N, K), device="cuda", generator=g, dtype=torch.int32).to(torch.int8)
    sw = torch.rand(K // 128, N, device="cuda", generator=g) * 0.01 + 0.001
    wq_t = wq.view(N, K // 16, 16).permute(1, 0, 2).contiguous()
    x = torch.randn(M, K, device="cuda", generator=g).to(torch.bfloat16)
    xq, xs = ext.w8a16_quant_act(x)
    amax = x.float().abs().amax(1)
    assert torch.allclose(xs, (amax / 127).clamp_min(1e-12), rtol=1e-6)
    assert (xq.float() * xs[:, None] - x.float()).abs().max() <= xs.max() * 0.51
    y = ext.w8a16_gemm(xq, xs, wq_t, sw, N, K, S)
    part = (xq.double().view(M, K // 128, 128)[:, :, None, :] * wq.double().view(N, K // 128, 128).permute(1, 0, 2)[None]).sum(-1)
    want = (part * sw.double()[None]).sum(1) * xs.double()[:, None]
    assert rel_l2(y, want) < 2e-2


@pytest.mark.parametrize("m,n,k,group", [(1, 512, 3072, 128), (16, 5120, 5120, 128), (64, 3456, 5120, 128),
                                         (200, 640, 1024, 64), (8, 384, 1536, 256)])
def test_group_scales_inside_the_kernel(ext, m, n, k, group):
    """Per-group scales (the reference kernel's granularity) applied while the tile is widened:
    against fp64 on the quantised operands, the reference's criterion."""
    from barlink_sm86_b200 import ops
    from barlink_sm86_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(11)
    w = torch.randn(n, k, device="cuda", generator=g) * 0.02
    w[:, : k // 2] *= 7.0   # groups of one row differ by an order of magnitude
    wq, scale = ref.quantize_w8_grouped(w, group)
    x = torch.randn(m, k, device="cuda", generator=g).to(torch.bfloat16)
    gs = ops.prepare_w8_scales(scale, k)
    got = ops.w8a16_linear(x, wq, gs)
    got2 = ops.w8a16_linear(x, wq, scale)   # raw 2-D scales: prepared on the fly, same kernel
    torch.cuda.synchronize()
    assert ext.w8_error_flag(0) == 0
    want = x.double() @ ref.w8_dequant(wq, scale).double().t()
    assert rel_l2(got, want) < 2e-2, (m, n, k, group)
    assert torch.equal(got, got2)


def test_prefill_dequant_then_gemm_has_no_weight_prefetch_race(ext):
    """More than 256 tokens: the weight is widened into a fresh buffer and the bf16 GEMM runs on
    it.  The GEMM must not request weight tiles before the widening kernel has finished: a large
    weight on a reused, garbage-filled buffer, many times."""
    from barlink_sm86_b200.ops import reference as ref
    n, k, m = 18944, 3584, 512
    wq, scale = _quant(n, k, 21)
    x = torch.randn(m, k, device="cuda", generator=torch.Generator("cuda").manual_seed(22)).to(torch.bfloat16)
    want = ref.w8a16_linear(x, wq, scale)
    for it in range(6):
        junk = torch.full((n, k), float("nan"), dtype=torch.bfloat16, device="cuda")  # the allocator hands this block back
        del junk
        got = ext.w8a16_linear(x, wq, scale)
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all(), it
        assert rel_l2(got, want) < 1.5e-2, it
