# SPDX-License-Identifier: MIT
"""One gloo rank of the CPU process-group test (started by test_pg_cpu.py)."""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
os.environ["BL_CPU_ONLY"] = "1"

from barlink_sm86_b200 import process_group as blpg  # noqa: E402

mode, rank, world, port = sys.argv[1], int(sys.argv[2]), int(sys.argv[3]), int(sys.argv[4])
if mode == "late" and rank == 1:
    sys.exit(0)  # this rank never joins: the others must fail with a timeout, not hang
try:
    from datetime import timedelta
    blpg.init_process_group(init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world,
                            timeout=timedelta(seconds=8 if mode == "late" else 120))
except Exception as e:
    if mode == "late":
        print("rendezvous failed as expected: %s" % type(e).__name__)
        sys.exit(3)
    raise

if mode == "collectives":
    t = torch.full((7,), float(rank + 1))
    dist.all_reduce(t)
    assert torch.all(t == sum(range(1, world + 1)))
    m = torch.tensor([float(rank)])
    dist.all_reduce(m, op=dist.ReduceOp.MAX)
    assert m.item() == world - 1
    out = torch.empty(world * 3)
    dist.all_gather_into_tensor(out, torch.full((3,), float(rank)))
    assert torch.equal(out, torch.arange(world).repeat_interleave(3).float())
    part = torch.empty(2)
    dist.reduce_scatter_tensor(part, torch.arange(2. * world))
    assert torch.equal(part, torch.arange(2. * world)[2 * rank:2 * rank + 2] * world)
    b = torch.arange(5.) if rank == 0 else torch.zeros(5)
    dist.broadcast(b, src=0)
    assert torch.equal(b, torch.arange(5.))
    if rank == 0:
        dist.send(torch.tensor([42.]), 1)
    elif rank == 1:
        r = torch.zeros(1)
        dist.recv(r, 0)
        assert r.item() == 42.
    dist.barrier()
    subs = [dist.new_group([r]) for r in range(world)]
    s = torch.tensor([float(rank)])
    dist.all_reduce(s, group=subs[rank])
    assert s.item() == float(rank)
    import torch.distributed._functional_collectives as fc
    y = fc.all_reduce(torch.ones(3), "sum", dist.group.WORLD)
    assert torch.all(y == world)
    be = blpg.backend_of()
    assert type(be).__name__ == "BarlinkBackend" and be.n_cpu > 0
    # a CUDA-free group must refuse CUDA tensors with a clear message (not reachable here without a GPU)
elif mode == "tiny":
    from barlink_sm86_b200.models import Qwen2Config, Qwen2Model
    from barlink_sm86_b200.parallel import TPComm
    cfg = Qwen2Config.tiny()
    ids = torch.randint(0, cfg.vocab, (2, 128), generator=torch.Generator().manual_seed(1), dtype=torch.int32)
    tp = Qwen2Model(cfg, TPComm(dist.group.WORLD), "cpu", torch.float32, seed=0)
    one = Qwen2Model(cfg, TPComm.single(), "cpu", torch.float32, seed=0)
    lt, l1 = tp.logits(tp.prefill(ids)), one.logits(one.prefill(ids))
    err = (lt - l1).abs().max().item()
    print("tiny TP=%d max abs logit error %.2e" % (world, err))
    assert err < 1e-4, err
    nt, n1 = tp.next_tokens(tp.prefill(ids)), one.next_tokens(one.prefill(ids))
    assert torch.equal(nt, n1)
    # quantised weights: a shard quantises to the same values as the unsharded rows, so TP stays exact;
    # against the unquantised model the logits only have to stay close
    for quant in ("w8a16", "w4a16"):
        qt = Qwen2Model(cfg, TPComm(dist.group.WORLD), "cpu", torch.float32, seed=0, quant=quant)
        q1 = Qwen2Model(cfg, TPComm.single(), "cpu", torch.float32, seed=0, quant=quant)
        a, b = qt.logits(qt.prefill(ids[:1, :32])), q1.logits(q1.prefill(ids[:1, :32]))
        ref_l = one.logits(one.prefill(ids[:1, :32]))
        err = (a - b).abs().max().item()
        cos = torch.cosine_similarity(b.flatten(), ref_l.flatten(), dim=0).item()
        print("tiny %s TP=%d max abs logit error %.2e, cosine vs unquantised %.4f" % (quant, world, err, cos))
        assert err < 1e-3 and cos > (0.99 if quant == "w8a16" else 0.9), (quant, err, cos)
elif mode == "checkpoint":
    # export a random model as a Hugging Face style checkpoint (rank 0), load it back sharded on every rank
    import tempfile
    from barlink_sm86_b200.models import Qwen2Config, Qwen2Model
    from barlink_sm86_b200.parallel import TPComm
    from barlink_sm86_b200.utils import SafetensorsSource, save_qwen2_safetensors
    cfg = Qwen2Config.tiny()
    one = Qwen2Model(cfg, TPComm.single(), "cpu", torch.float32, seed=4)
    for L in one.w.layers:  # norm weights other than one, so that a swapped norm would show
        L["ln1"].uniform_(0.5, 1.5, generator=torch.Generator().manual_seed(1))
        L["ln2"].uniform_(0.5, 1.5, generator=torch.Generator().manual_seed(2))
    d = os.path.join(tempfile.gettempdir(), "bl-ckpt-test-%d" % port)
    if rank == 0:
        save_qwen2_safetensors(one, d, shard_bytes=4 << 20)   # several shards
    dist.barrier()
    src = SafetensorsSource(d, "cpu", torch.float32)
    c2 = src.config()
    assert (c2.hidden, c2.layers, c2.n_heads, c2.n_kv_heads, c2.head_dim, c2.intermediate, c2.vocab, c2.qkv_bias) == \
        (cfg.hidden, cfg.layers, cfg.n_heads, cfg.n_kv_heads, cfg.head_dim, cfg.intermediate, cfg.vocab, cfg.qkv_bias)
    tp = Qwen2Model(c2, TPComm(dist.group.WORLD), "cpu", torch.float32, source=src)
    ids = torch.randint(0, cfg.vocab, (2, 24), generator=torch.Generator().manual_seed(3), dtype=torch.int32)
    err = (tp.logits(tp.prefill(ids)) - one.logits(one.prefill(ids))).abs().max().item()
    print("checkpoint round trip TP=%d max abs logit error %.2e" % (world, err))
    assert err < 1e-4, err
    dist.barrier()
    if rank == 0:
        import shutil
        shutil.rmtree(d, ignore_errors=True)
elif mode == "mmdit":
    from barlink_sm86_b200.models import MMDiTConfig, MMDiTModel, MMDiTWeights, grid_positions
    from barlink_sm86_b200.parallel import TPComm
    cfg = MMDiTConfig.tiny()
    g = torch.Generator().manual_seed(5)
    img = torch.randn(2, 16, cfg.in_channels, generator=g)
    txt = torch.randn(2, 8, cfg.txt_dim, generator=g)
    t = torch.tensor([0.9, 0.3])
    pos = grid_positions(4, 4, "cpu")
    tp = MMDiTModel(cfg, MMDiTWeights(cfg, "cpu", torch.float32, 0, world, rank), TPComm(dist.group.WORLD))
    one = MMDiTModel(cfg, MMDiTWeights(cfg, "cpu", torch.float32, 0), TPComm.single())
    yt, y1 = tp.forward(img, txt, t, pos), one.forward(img, txt, t, pos)
    err = ((yt - y1).norm() / y1.norm()).item()
    print("tiny MMDiT TP=%d rel-L2 vs one rank %.2e" % (world, err))
    assert err < 1e-4, err
elif mode == "raise":
    # a rank that raises between steps: the others learn of it on the host
    store = dist.distributed_c10d._get_default_store()
    if rank == 1:
        store.set("failed/1", "boom")
        dist.destroy_process_group()
        sys.exit(7)
    store.wait(["failed/1"])
    print("rank %d saw the failure of rank 1" % rank)
dist.barrier() if mode != "raise" else None
if mode != "raise":
    dist.destroy_process_group()
