#!/usr/bin/env python
# SPDX-License-Identifier: MIT
"""Phase stamps of the decode linears (`_C.dlin`, csrc/dlin_kernels.cu) on one GPU: every CTA
records the global timer at fixed points (start, barriers and TMEM ready, dependency wait passed,
activation rows published, first MMA, last MMA issued, gather done, accumulator ready, partials
handed over through distributed shared memory, cluster barrier passed, end) and the script prints
the median and the maximum over the CTAs, relative to the first CTA's start, for the four linears
of a TP=8 shard of the 7B shape at 64 tokens and several cluster sizes.  L2 is flushed before the
traced launch (cold weights, as in the decode step, and cold activations, unlike it).

    python bench/gemm/dlin_phases.py

The reference has no counterpart (its linears are library calls)."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
import barlink_sm86_b200 as bl
from barlink_sm86_b200 import ops
C = bl.load_extension()
torch.manual_seed(0)
T, H = 64, 3584
def bf(*s): return (torch.randn(*s, device='cuda') * 0.05).bfloat16()
flush = torch.empty(256 << 20, dtype=torch.uint8, device='cuda')
names = ["start", "setup", "pdl_wait", "gate", "mma0", "mma_end", "pro_end", "tfull", "scatter", "csync", "end"]
link = C.dlin_local_link(T, H, 0)
res = bf(T, H); xn = torch.zeros(T, H, dtype=torch.bfloat16, device='cuda'); gamma = torch.ones(H, dtype=torch.bfloat16, device='cuda')
wo = bf(H, 512); a_in = bf(T, 512)
def show(tag, n, k, cl, run):
    clu = C.dlin_cluster(n, k, T, cl)
    grid = ((n + 127) // 128) * clu
    tr = torch.zeros(12 * 8 * ((n + 127) // 128), dtype=torch.int64, device='cuda')
    for _ in range(2): run(None)
    flush.zero_(); torch.cuda.synchronize()
    run(tr); torch.cuda.synchronize()
    t_ = tr[:12 * grid].view(grid, 12).cpu().double()
    t0 = t_[:, 0].min()
    rel = (t_ - t0) / 1e3
    med = [rel[:, i][t_[:, i] > 0].median().item() if (t_[:, i] > 0).any() else float('nan') for i in range(11)]
    mx = [rel[:, i][t_[:, i] > 0].max().item() if (t_[:, i] > 0).any() else float('nan') for i in range(11)]
    print("  %s cluster %d (grid %d): total %.1f us | median: %s" % (tag, clu, grid, mx[10], " ".join("%s=%.1f" % (a, b) for a, b in zip(names, med))))
    print("      max: %s" % " ".join("%s=%.1f" % (a, b) for a, b in zip(names, mx)))
for name, n, k, epi in [("o_proj", 3584, 512, "push"), ("down", 3584, 2368, "push"), ("gate_up", 4736, 3584, "silu_mul"), ("qkv", 768, 3584, "store")]:
    w, x = bf(n, k), bf(T, k)
    print("== %s n=%d k=%d" % (name, n, k))
    for cl in (0, 1, 2, 3, 4, 5, 8):
        if epi == "push":
            def run(tr):
                C.dlin(x, w, epi="push", hidden=H, link=link, cluster=cl, trace=tr)
                C.gather_norm(xn, res, gamma, 1e-6, link=link)
            show("push", n, k, cl, run)
        else:
            show("plain", n, k, cl, lambda tr: C.dlin(x, w, epi=epi, cluster=cl, trace=tr))
            def run(tr):
                C.dlin(a_in, wo, epi="push", hidden=H, link=link)
                C.dlin(xn, w, pro="gather_norm", epi=epi, residual=res, gamma=gamma, eps=1e-6, link=link, cluster=cl, trace=tr)
            show("gather+norm prologue", n, k, cl, run)
print("dlin_error_flag", C.dlin_error_flag(0))
