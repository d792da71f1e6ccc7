# SPDX-License-Identifier: MIT
"""Smallest end-to-end check of the decode path on one device: a tiny decoder,
prefill + a few greedy steps, eager against the captured graph (on CUDA) and
every weight format.  Counterpart of demos/qwen_tp/qwen38_int8/smoke.py."""
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))
from barlink_sm86_b200.models import DecodeEngine, Qwen2Config, Qwen2Model  # noqa: E402
from barlink_sm86_b200.parallel import TPComm  # noqa: E402

cuda = torch.cuda.is_available()
dev, dt = ("cuda:0", torch.bfloat16) if cuda else ("cpu", torch.float32)
cfg = Qwen2Config(hidden=1024, layers=2, n_heads=8, n_kv_heads=2, head_dim=128, intermediate=2816,
                  vocab=4096, name="smoke")
ids = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(0), dtype=torch.int32).to(dev)
for quant in ("none", "w8a16", "w4a16"):
    outs = []
    for graph in ((False, True) if cuda else (False,)):
        m = Qwen2Model(cfg, TPComm.single(), dev, dt, seed=1, quant=quant)
        e = DecodeEngine(m, 2, 64, use_graph=graph)
        e.ids.copy_(e.prefill(ids))
        e.capture()
        outs.append(torch.stack([e.step().clone() for _ in range(6)], 1).cpu())
    assert all(torch.equal(outs[0], o) for o in outs[1:]), "graph replay differs from eager (%s)" % quant
    print("%-6s tokens %s" % (quant, outs[0][0].tolist()))
print("SMOKE OK on", dev)
