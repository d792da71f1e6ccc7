# SPDX-License-Identifier: MIT
"""One rank of the tensor-parallel model test (started by test_pg_gpu.py):
TP=N logits against the TP=1 model held on the same GPU, and greedy decode
through the CUDA-graphed engine with identical tokens on every rank (the
reference's compare.py checks: demos/qwen_tp/qwen38_int8/compare.py:44-74)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200 import process_group as blpg  # noqa: E402
from barlink_sm86_b200.models import DecodeEngine, Qwen2Config, Qwen2Model  # noqa: E402
from barlink_sm86_b200.parallel import TPComm  # noqa: E402

rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
os.environ["LOCAL_RANK"] = str(rank)
os.environ.setdefault("BL_POOL_MB", "512")
os.environ["BL_DLIN"] = "auto"     # the folded-collective decode path (whatever the library's default is)
os.environ["BL_PUSH_AR"] = "1"     # prefill: row-parallel linears that scatter their tiles themselves
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
blpg.init_process_group(init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)

cfg = Qwen2Config(hidden=1024, layers=3, n_heads=8, n_kv_heads=2, head_dim=128, intermediate=2816,
                  vocab=4096, name="tp-test")
tp = Qwen2Model(cfg, TPComm(dist.group.WORLD), dev, torch.bfloat16, seed=9)
one = Qwen2Model(cfg, TPComm.single(), dev, torch.bfloat16, seed=9)
B, S, steps = max(4, world), 40, 8  # B % world == 0 (token-sharded paths); B * S > 128: prefill takes the pushed row-parallel linears
ids = torch.randint(0, cfg.vocab, (B, S), generator=torch.Generator().manual_seed(5), dtype=torch.int32).to(dev)
lt = tp.logits(tp.prefill(ids)).float()
l1 = one.logits(one.prefill(ids)).float()
rel = ((lt - l1).norm() / l1.norm()).item()
assert rel < 3e-2, rel


def generate(model):
    eng = DecodeEngine(model, B, S + steps + 8, use_graph=True)
    first = eng.prefill(ids)
    eng.ids.copy_(first)
    eng.capture()
    seq = [first.clone()]
    for _ in range(steps):
        seq.append(eng.step().clone())
    return torch.stack(seq, 1)


# default: one kernel per linear with the all-reduce halves folded into epilogue and prologue
assert tp.dlin_ok(B), "the folded-collective decode path should be available for this shape"
tok_tp = generate(tp)
os.environ["BL_DLIN"] = "0"
os.environ["BL_FUSED_LINEAR"] = "1"
assert tp.fused_ok(B), "the fused TP linears should be available for this shape"
tok_rs = generate(tp)
os.environ["BL_FUSED_LINEAR"] = "0"
tok_unfused = generate(tp)
os.environ["BL_DLIN"] = "auto"
tok_1 = generate(one)
m_fu = (tok_tp == tok_unfused).float().mean().item()
m_rs = (tok_rs == tok_unfused).float().mean().item()
if rank == 0:
    print("[tp] token match with the all-reduce path: folded %.0f%%, reduce-scatter/all-gather %.0f%%"
          % (m_fu * 100, m_rs * 100), flush=True)
assert m_fu >= 0.7, m_fu
assert m_rs >= 0.7, m_rs
assert bl.load_extension().dlin_error_flag(rank) == 0
gathered = [torch.empty_like(tok_tp) for _ in range(world)]
dist.all_gather(gathered, tok_tp)
for g in gathered:
    assert torch.equal(g, tok_tp), "ranks disagree on the generated tokens"
match = (tok_tp == tok_1).float().mean().item()
if rank == 0:
    print("[tp] world %d logits rel-L2 %.4f, token match vs TP=1 %.0f%%, all-reduce calls %d"
          % (world, rel, match * 100, tp.comm.ar_calls), flush=True)
assert match >= 0.7, match
assert bl.status()["code"] == 0
dist.barrier()
dist.destroy_process_group()
bl.shutdown()
