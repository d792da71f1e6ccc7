# SPDX-License-Identifier: MIT
"""MMDiT kernels and model on one GPU against their fp32 PyTorch statements."""
import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,heads,extra,axes,norm", [(37, 3, 128, 2, True), (64, 24, 0, 2, True),
                                                        (5, 2, 512, 1, False), (130, 6, 384, 1, True)])
def test_qknorm_rope(ext, rows, heads, extra, axes, norm):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(rows)
    width = 3 * heads * 128 + extra
    qkv = torch.randn(rows, width, generator=g).bfloat16()
    gq = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16() if norm else None
    gk = (1 + 0.1 * torch.randn(128, generator=g)).bfloat16() if norm else None
    pos = torch.randint(0, 64, (rows, axes), generator=g, dtype=torch.int32)
    want = ops.ref.qknorm_rope(qkv.clone(), gq, gk, pos, heads, 1e-6, 1e4, axes)
    got = ops.qknorm_rope(qkv.cuda(), gq.cuda() if norm else None, gk.cuda() if norm else None, pos.cuda(),
                          heads, 1e-6, 1e4, axes).cpu()
    assert rel_l2(got[:, : 2 * heads * 128], want[:, : 2 * heads * 128]) < 1e-2
    assert torch.equal(got[:, 2 * heads * 128:], qkv[:, 2 * heads * 128:])  # v and the rest untouched


@pytest.mark.parametrize("batch,per,hidden", [(1, 33, 3072), (3, 17, 256), (2, 64, 1024)])
def test_layernorm_modulate_and_gate_residual(ext, batch, per, hidden):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(hidden)
    x = torch.randn(batch * per, hidden, generator=g).bfloat16()
    mod = (0.3 * torch.randn(batch, 3 * hidden, generator=g)).bfloat16()
    sh, sc, gt = (mod[:, j * hidden:(j + 1) * hidden] for j in range(3))
    want = ops.ref.layernorm_modulate(x, sh, sc, per)
    mg = mod.cuda()
    shg, scg, gtg = (mg[:, j * hidden:(j + 1) * hidden] for j in range(3))
    got = ops.layernorm_modulate(x.cuda(), shg, scg, per).cpu()
    assert rel_l2(got, want) < 1e-2
    y = torch.randn(batch * per, hidden, generator=g).bfloat16()
    want = ops.ref.gate_residual(x.clone(), y, gt, per)
    got = ops.gate_residual(x.cuda(), y.cuda(), gtg, per).cpu()
    assert rel_l2(got, want) < 1e-2


@pytest.mark.parametrize("m,n,k", [(300, 512, 256), (8, 1024, 512), (1, 768, 256)])
def test_linear_gelu_epilogue(ext, m, n, k):
    from barlink_sm86_b200 import ops
    g = torch.Generator().manual_seed(m)
    x = torch.randn(m, k, generator=g).bfloat16()
    w = (torch.randn(n, k, generator=g) / k ** 0.5).bfloat16()
    b = torch.randn(n, generator=g).bfloat16()
    want = ops.ref.linear(x, w, b, gelu=True)
    got = ops.linear(x.cuda(), w.cuda(), b.cuda(), gelu=True).cpu()
    assert rel_l2(got, want) < 1e-2
    assert ext.gemm_error_flag(0) == 0


@pytest.mark.parametrize("batch", [1, 2])
def test_tiny_mmdit_matches_fp32_cpu_model(ext, batch):
    from barlink_sm86_b200.models import MMDiTConfig, MMDiTModel, MMDiTWeights, grid_positions
    cfg = MMDiTConfig.tiny(hidden=512, heads=4)
    g = torch.Generator().manual_seed(11)
    img = torch.randn(batch, 96, cfg.in_channels, generator=g).bfloat16()
    txt = torch.randn(batch, 40, cfg.txt_dim, generator=g).bfloat16()
    t = torch.linspace(0.8, 0.2, batch)
    pos = grid_positions(8, 12, "cpu")
    gpu = MMDiTModel(cfg, MMDiTWeights(cfg, "cuda:0", torch.bfloat16, 2, gen_device="cpu"))
    cpu = MMDiTModel(cfg, MMDiTWeights(cfg, "cpu", torch.bfloat16, 2, gen_device="cpu"))
    # the CPU model holds the same bf16 values but computes every op in fp32
    got = gpu.forward(img.cuda(), txt.cuda(), t.cuda(), pos.cuda()).float().cpu()
    want = cpu.forward(img, txt, t, pos).float()
    assert rel_l2(got, want) < 5e-2
    assert ext.gemm_error_flag(0) == 0
