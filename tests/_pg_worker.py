# SPDX-License-Identifier: MIT
"""One rank of the multi-GPU process-group test (started by test_pg_gpu.py).

Same fixtures as the reference's distributed tests
(torch_ext/tests/test_process_group.py:24-197, test_pg_p2p.py:42-245,
test_pg_gather.py:24-62): rank-seeded data so that every rank can compute the
expected result locally, and argument errors that must be raised before any
traffic so that a failing check cannot desynchronise the ranks."""
import os
import sys
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

import barlink_sm86_b200 as bl  # noqa: E402
from barlink_sm86_b200 import process_group as blpg  # noqa: E402

rank, world, port = int(sys.argv[1]), int(sys.argv[2]), int(sys.argv[3])
os.environ["LOCAL_RANK"] = str(rank)
os.environ.setdefault("BL_POOL_MB", "512")
torch.cuda.set_device(rank)
dev = torch.device("cuda", rank)
blpg.init_process_group(init_method="tcp://127.0.0.1:%d" % port, rank=rank, world_size=world)
C = bl.load_extension()
info = bl.info()
assert info["peer_mode"] and info["world"] == world and info["rank"] == rank, info


def log(msg):
    if rank == 0:
        print("[pg] " + msg, flush=True)


def seeded(r, n, dtype, lo=-3, hi=4):
    g = torch.Generator(device="cpu").manual_seed(1000 + r)
    return torch.randint(lo, hi, (n,), generator=g).to(dtype)


def expect_sum(n, dtype):
    acc = torch.zeros(n, dtype=torch.float64)
    for r in range(world):
        acc += seeded(r, n, torch.float64)
    return acc.to(dtype)


def host_barrier():
    t = torch.zeros(1)
    dist.all_reduce(t)  # CPU tensor: gloo companion


# ---- proof of every path ------------------------------------------------------
assert bl.verify() == 0
log("verify ok (multicast=%s)" % info["multicast"])

# ---- all_reduce: sizes, dtypes, algorithms ------------------------------------------
for nbytes in (1024, 1 << 20, 32 << 20, (96 << 20) + 16):
    n = nbytes // 4
    t = seeded(rank, n, torch.float32).to(dev)
    dist.all_reduce(t)
    assert torch.equal(t.cpu(), expect_sum(n, torch.float32)), nbytes
log("all_reduce sizes ok")
for dtype in (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.float8_e4m3fn,
              torch.float8_e5m2):
    n = 4096
    t = seeded(rank, n, torch.float32).to(dtype).to(dev)
    dist.all_reduce(t)
    assert torch.equal(t.cpu().view(torch.uint8), expect_sum(n, torch.float32).to(dtype).view(torch.uint8)), dtype
u = torch.arange(4096, dtype=torch.int64).mul(rank + 7).remainder(256).to(torch.uint8).to(dev)
dist.all_reduce(u)
want = sum(torch.arange(4096, dtype=torch.int64).mul(r + 7).remainder(256) for r in range(world)).remainder(256)
assert torch.equal(u.cpu().long(), want)
log("all_reduce dtypes ok")
algos = ["oneshot", "twoshot"] + (["nvls"] if info["multicast"] else [])
for algo in algos:
    for nbytes in (16, 10240, 256 << 10, 4 << 20):
        n = nbytes // 2
        x = seeded(rank, n, torch.bfloat16).to(dev)
        out = torch.empty_like(x)
        bl.allreduce_into(out, x, algo)
        assert torch.equal(out.cpu(), expect_sum(n, torch.bfloat16)), (algo, nbytes)
log("all_reduce algorithms ok: %s" % algos)
if info["multicast"]:
    # in-switch reduction on a bandwidth-sized message, integer-valued so that the sum is exact
    for nbytes, dtype in ((64 << 20, torch.bfloat16), (16 << 20, torch.float32)):
        nbytes = min(nbytes, info["max_chunk"])   # one call's limit depends on the arena and the ranks
        n = nbytes // torch.empty(0, dtype=dtype).element_size()
        x = seeded(rank, n, dtype).to(dev)
        out = torch.empty_like(x)
        bl.allreduce_into(out, x, "nvls")
        assert torch.equal(out.cpu(), expect_sum(n, dtype)), ("nvls", nbytes, dtype)
    log("nvls large messages ok")

# back-to-back staged collectives with a different pattern per call, while one rank's SMs are
# also busy with an unrelated stream: a call must never overwrite staging data that a slower
# peer has not consumed yet
side = torch.cuda.Stream()
busy_a = torch.randn(2048, 2048, device=dev)
stop_at = 120
n = 96 << 10
mine_all = [seeded(rank, n, torch.float32).add(i).to(dev) for i in range(4)]
for it in range(stop_at):
    if rank == 1 and it % 4 == 0:
        with torch.cuda.stream(side):
            for _ in range(6):
                busy_a = (busy_a @ busy_a).clamp_(-1, 1)
    mine = mine_all[it % 4]
    out = torch.empty(world * n, dtype=torch.float32, device=dev)
    dist.all_gather_into_tensor(out, mine)
    big = out  # every rank now holds the same [world * n] tensor
    part = torch.empty(n, dtype=torch.float32, device=dev)
    dist.reduce_scatter_tensor(part, big)
    if it % 10 == 0 or it == stop_at - 1:
        want_g = torch.cat([seeded(r, n, torch.float32).add(it % 4) for r in range(world)])
        assert torch.equal(out.cpu(), want_g), ("all_gather", it)
        assert torch.equal(part.cpu(), want_g[rank * n:(rank + 1) * n] * world), ("reduce_scatter", it)
torch.cuda.synchronize()
assert bl.status()["code"] == 0
log("back-to-back all_gather / reduce_scatter ok (%d rounds)" % stop_at)

# staged paths: odd size, unaligned view, non-contiguous
t = seeded(rank, 1001, torch.float32).to(dev)
dist.all_reduce(t)
assert torch.equal(t.cpu(), expect_sum(1001, torch.float32))
base = seeded(rank, 4100, torch.float16).to(dev)
v = base[1:4098]
dist.all_reduce(v)
assert torch.equal(v.cpu(), expect_sum(4100, torch.float16)[1:4098])
m = seeded(rank, 64 * 64, torch.float32).view(64, 64).to(dev)
mt = m.t()
dist.all_reduce(mt)
assert torch.equal(mt.cpu(), expect_sum(64 * 64, torch.float32).view(64, 64).t())
be = blpg.backend_of()
assert be.n_staged >= 3 and be.n_zero_copy > 0
log("staged fallbacks ok (zero-copy %d, staged %d)" % (be.n_zero_copy, be.n_staged))

# reuse loop on the decode message size, bitwise check every 50
n = 5120
for it in range(300):
    t = (seeded(rank, n, torch.float32) + it).to(torch.bfloat16).to(dev) if it % 50 == 0 else t
    if it % 50 == 0:
        keep = t.clone()
    dist.all_reduce(t)
    if it % 50 == 0:
        want = sum((seeded(r, n, torch.float32) + it).to(torch.bfloat16).float() for r in range(world)).to(torch.bfloat16)
        assert torch.equal(t.cpu(), want), it
assert bl.status()["code"] == 0
log("soak ok")

# ---- gather / scatter / broadcast / barrier ----------------------------------------
n = 2560
mine = seeded(rank, n, torch.bfloat16).to(dev)
out = torch.empty(world * n, dtype=torch.bfloat16, device=dev)
dist.all_gather_into_tensor(out, mine)
assert torch.equal(out.cpu(), torch.cat([seeded(r, n, torch.bfloat16) for r in range(world)]))
lst = [torch.empty(333, dtype=torch.float32, device=dev) for _ in range(world)]
dist.all_gather(lst, seeded(rank, 333, torch.float32).to(dev))
for r in range(world):
    assert torch.equal(lst[r].cpu(), seeded(r, 333, torch.float32))
big = seeded(rank, world * 4096, torch.float32).to(dev)
part = torch.empty(4096, dtype=torch.float32, device=dev)
dist.reduce_scatter_tensor(part, big)
assert torch.equal(part.cpu(), expect_sum(world * 4096, torch.float32)[rank * 4096:(rank + 1) * 4096])
for root in range(world):
    t = seeded(rank, 9999, torch.float32).to(dev)
    dist.broadcast(t, src=root)
    assert torch.equal(t.cpu(), seeded(root, 9999, torch.float32))
dist.barrier()
log("gather/scatter/broadcast/barrier ok")

# groups of one member are local no-ops and leave the world group intact
subs = [dist.new_group([r]) for r in range(world)]
t = torch.full((8,), float(rank), device=dev)
dist.all_reduce(t, group=subs[rank])
assert torch.all(t == float(rank))
t = torch.ones(64, device=dev)
dist.all_reduce(t)
assert torch.all(t == world)
log("size-1 groups ok")

# ---- p2p ---------------------------------------------------------------------------------
peer = rank ^ 1
if peer < world:
    for nbytes in (1024, 64 << 10, 8 << 20, 1000):
        n = nbytes // 4
        a = seeded(rank, n, torch.float32).to(dev)
        b = torch.empty(n, dtype=torch.float32, device=dev)
        reqs = [dist.isend(a, peer), dist.irecv(b, peer)]
        for r in reqs:
            r.wait()
        assert torch.equal(b.cpu(), seeded(peer, n, torch.float32)), nbytes
    # three sends outstanding before the first recv
    outs = [seeded(rank, 2048, torch.float32).add(i).to(dev) for i in range(3)]
    ins = [torch.empty(2048, dtype=torch.float32, device=dev) for _ in range(3)]
    for o in outs:
        dist.send(o, peer)
    for i in ins:
        dist.recv(i, peer)
    for i, t in enumerate(ins):
        assert torch.equal(t.cpu(), seeded(peer, 2048, torch.float32).add(i))
    # ping-pong
    t = torch.zeros(2560, device=dev)
    for it in range(20):
        if rank < peer:
            t.fill_(it)
            dist.send(t, peer)
            dist.recv(t, peer)
            assert torch.all(t == it + 0.5)
        else:
            dist.recv(t, peer)
            t.add_(0.5)
            dist.send(t, peer)
    log("p2p ok")

# every pair, several dtypes: rank r sends to r + d and receives from r - d (the reference's
# matrix for two ranks, torch_ext/tests/test_pg_p2p.py:143-206, over all distances of N ranks)
for d in range(1, world):
    to, frm = (rank + d) % world, (rank - d) % world
    for dtype, n in ((torch.float16, 4096), (torch.uint8, 40000), (torch.int64, 777), (torch.float32, 2 << 20)):
        a = seeded(rank, n, torch.float32, 0, 100).to(dtype).to(dev)
        b = torch.empty(n, dtype=dtype, device=dev)
        reqs = [dist.isend(a, to), dist.irecv(b, frm)]
        for r in reqs:
            r.wait()
        assert torch.equal(b.cpu(), seeded(frm, n, torch.float32, 0, 100).to(dtype)), (d, dtype)
# several sends of mixed sizes outstanding before the first receive is posted, all-reduces before
# and after; then p2p and all-reduce strictly interleaved (a collective on the caller's stream
# waits for the sends queued so far, so it may only follow sends whose receives are already posted
# on the peer -- the same rule NCCL imposes)
to, frm = (rank + 1) % world, (rank - 1) % world
sizes = (10, 70000, 3, 1 << 20)
outs = [seeded(rank, n, torch.float32).add(i).to(dev) for i, n in enumerate(sizes)]
ins = [torch.empty(n, dtype=torch.float32, device=dev) for n in sizes]
t = torch.ones(2560, dtype=torch.bfloat16, device=dev)
dist.all_reduce(t)
assert torch.all(t == world)
pend = [dist.isend(o, to) for o in outs] + [dist.irecv(buf, frm) for buf in ins]
for r in pend:
    r.wait()
t = torch.ones(1 << 20, device=dev)
dist.all_reduce(t)
assert torch.all(t == world)
for i, (buf, n) in enumerate(zip(ins, sizes)):
    assert torch.equal(buf.cpu(), seeded(frm, n, torch.float32).add(i)), ("mixed", i)
for i, n in enumerate(sizes):
    o = seeded(rank, n, torch.float32).add(10 + i).to(dev)
    buf = torch.empty(n, dtype=torch.float32, device=dev)
    reqs = [dist.isend(o, to), dist.irecv(buf, frm)]
    t = torch.full((4096,), float(i), dtype=torch.bfloat16, device=dev)
    dist.all_reduce(t)
    for r in reqs:
        r.wait()
    assert torch.all(t == float(i * world)), ("interleaved all_reduce", i)
    assert torch.equal(buf.cpu(), seeded(frm, n, torch.float32).add(10 + i)), ("interleaved", i)
# a message far above the p2p slice goes in chunks, full duplex (reference: repro_p2p_big.py:23-71)
for mb in (48, 128):
    n = (mb << 20) // 4
    a = torch.arange(n, dtype=torch.int32, device=dev).mul_(rank + 3)
    b = torch.empty(n, dtype=torch.int32, device=dev)
    reqs = [dist.isend(a, to), dist.irecv(b, frm)]
    for r in reqs:
        r.wait()
    assert torch.equal(b, torch.arange(n, dtype=torch.int32, device=dev).mul_(frm + 3)), mb
# host tensors and a strided view take the staged fallback
hs = seeded(rank, 500, torch.float32)
hr = torch.empty(500)
reqs = [dist.isend(hs, to), dist.irecv(hr, frm)]
for r in reqs:
    r.wait()
assert torch.equal(hr, seeded(frm, 500, torch.float32))
base = seeded(rank, 4000, torch.float32).to(dev)
rb = torch.zeros(4000, device=dev)
reqs = [dist.isend(base[::2], to), dist.irecv(rb[::2], frm)]
for r in reqs:
    r.wait()
assert torch.equal(rb[::2].cpu(), seeded(frm, 4000, torch.float32)[::2]) and torch.all(rb[1::2] == 0)
log("p2p matrix ok (all distances, fp16/u8/int64/fp32, mixed with all-reduce, 48 and 128 MB, host and strided)")

# ---- fused all-reduce + residual + RMSNorm ------------------------------------------------
from barlink_sm86_b200.ops import reference as ref  # noqa: E402
for rows, hidden in ((1, 3584), (8, 3584), (64, 3584), (3, 5120)):
    g = torch.Generator(device="cpu").manual_seed(77)
    parts = [torch.randn(rows, hidden, generator=g).to(torch.bfloat16) for _ in range(world)]
    res = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    normed, new_res = bl.allreduce_rmsnorm(parts[rank].to(dev), res.to(dev), gamma.to(dev), 1e-6)
    want_n, want_r = ref.allreduce_rmsnorm(parts, res, gamma, 1e-6)
    assert torch.equal(new_res.cpu(), want_r)
    assert ((normed.cpu().float() - want_n.float()).norm() / want_n.float().norm()) < 5e-3
# the same with this rank's contribution given as k-split fp32 slabs of a linear
for rows, hidden, S in ((8, 3584, 4), (64, 3584, 5)):
    g = torch.Generator(device="cpu").manual_seed(78)
    slabs = [torch.randn(S, rows, hidden, generator=g) for _ in range(world)]
    parts = [s_.sum(0).to(torch.bfloat16) for s_ in slabs]
    res = torch.randn(rows, hidden, generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(torch.bfloat16)
    normed, new_res = bl.allreduce_rmsnorm(slabs[rank].to(dev), res.to(dev), gamma.to(dev), 1e-6)
    want_n, want_r = ref.allreduce_rmsnorm(parts, res, gamma, 1e-6)
    assert (new_res.cpu().float() - want_r.float()).abs().max() <= 0.07, "slab sum differs"
    assert ((normed.cpu().float() - want_n.float()).norm() / want_n.float().norm()) < 8e-3
log("allreduce_rmsnorm ok")

# ---- row-parallel linear whose epilogue is the scatter half of the all-reduce ------------------
from barlink_sm86_b200.parallel import TPComm  # noqa: E402
comm = TPComm(dist.group.WORLD)
for T, n, k, split in ((1024, 512, 256, 384), (world * 320, 768, 192, 0), (2304, 3072, 512, 256)):
    g = torch.Generator(device="cpu").manual_seed(4000 + rank)
    x = (torch.randn(T, k, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    w1 = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    w2 = (torch.randn(n, k, generator=g) * 0.05).to(torch.bfloat16).to(dev)
    bias = torch.randn(n, generator=g).to(torch.bfloat16).to(dev)
    res = torch.randn(T, n, generator=g).to(torch.bfloat16).to(dev)
    if split and T - split > 128 and split > 128:
        parts = [(x[:split], w1, bias, None, False, 0), (x[split:], w2, None, res[split:], True, split)]
    else:
        parts = [(x, w1, bias, res, False, 0)]
    os.environ["BL_PUSH_AR"] = "0"
    want = comm.row_parallel(torch.empty(T, n, dtype=torch.bfloat16, device=dev), parts).clone()
    # the statement of the operation: every rank's bf16 product, summed in fp32 in rank order, rounded once
    mine = torch.empty(T, n, dtype=torch.bfloat16, device=dev)
    for x_, w_, b_, r_, gelu_, row0_ in parts:
        # no k-split: the pushed GEMM has none either, and a k-split sums the products in another order
        C.linear(x_, w_, b_, r_, False, mine[row0_:row0_ + x_.shape[0]], splits=1, gelu=gelu_)
    every = torch.empty(world, T, n, dtype=torch.bfloat16, device=dev)
    dist.all_gather_into_tensor(every.view(-1), mine.view(-1))
    acc = torch.zeros(T, n, dtype=torch.float32, device=dev)
    for r_ in range(world):
        acc += every[r_].float()
    truth = acc.to(torch.bfloat16)
    # the plain path may k-split its GEMMs (each rank's bf16 product can then differ by one step of ITS
    # magnitude, which matters where the ranks' values cancel) and add in another order or in the switch
    step = torch.maximum(every.float().abs().amax(0), truth.float().abs()) * 2.0 ** -7
    off = (want.float() - truth.float()).abs()
    assert bool((off <= step * (world + 2)).all()), ("GEMM + all_reduce is off", T, n, k, off.max().item())
    os.environ["BL_PUSH_AR"] = "1"
    calls = bl.stats()["ops"]
    for it in range(3):   # consecutive calls alternate between the two staging buffers
        got = comm.row_parallel(torch.empty(T, n, dtype=torch.bfloat16, device=dev), parts)
        torch.cuda.synchronize()
        bad = (got != truth)
        assert not bool(bad.any()), ("pushed all-reduce differs from the rank-ordered fp32 sum", T, n, k, it,
                                     int(bad.sum()), (got.float() - truth.float()).abs().max().item(),
                                     bad.nonzero()[:4].tolist())
    assert bl.stats()["ops"] == calls + 3, "the pushed path did not run"
assert bl.status()["code"] == 0 and C.gemm_error_flag(rank) == 0
log("row-parallel linear with pushed all-reduce ok (bit-equal to the rank-ordered fp32 sum)")

# ---- CUDA graph capture and replay ----------------------------------------------------------
x = torch.zeros(5120, dtype=torch.bfloat16, device=dev)
y = torch.empty_like(x)
s = torch.cuda.Stream()
s.wait_stream(torch.cuda.current_stream())
with torch.cuda.stream(s):
    bl.allreduce_into(y, x)
torch.cuda.current_stream().wait_stream(s)
torch.cuda.synchronize()
g = torch.cuda.CUDAGraph()
with torch.cuda.graph(g):
    bl.allreduce_into(y, x)
    bl.allreduce_into(y, y, "twoshot")
for it in range(10):
    x.fill_(float(rank + it))
    g.replay()
    torch.cuda.synchronize()
    want = float(sum(r + it for r in range(world)) * world)
    assert torch.all(y.float() == want), (it, y[:4], want)
log("graph replay ok")

# ---- argument errors come before any traffic ------------------------------------------------
for op, want_fn in ((dist.ReduceOp.MAX, lambda v: max(v)), (dist.ReduceOp.MIN, lambda v: min(v)),
                    (dist.ReduceOp.AVG, lambda v: sum(v) / len(v)), (dist.ReduceOp.PRODUCT, None)):
    # non-SUM ops: gathered over the link and reduced locally (odd length: exercises the padding)
    t = torch.full((5,), float(rank + 2), device=dev)
    dist.all_reduce(t, op=op)
    vals = [float(r + 2) for r in range(world)]
    want = want_fn(vals) if want_fn else float(torch.tensor(vals).prod())
    assert torch.allclose(t, torch.full_like(t, want)), (op, t, want)
# a subgroup of 2 ranks inside a larger world: served through host memory by the gloo companion
if world >= 4:
    pairs = [dist.new_group([2 * i, 2 * i + 1]) for i in range(world // 2)]
    mine = pairs[rank // 2]
    t = torch.full((1000,), float(rank + 1), device=dev)
    dist.all_reduce(t, group=mine)
    lo = 2 * (rank // 2)
    assert torch.all(t == float(lo + 1 + lo + 2)), t[:4]
    gathered = torch.empty(2 * 8, device=dev)
    dist.all_gather_into_tensor(gathered, torch.full((8,), float(rank), device=dev), group=mine)
    assert torch.equal(gathered.cpu(), torch.tensor([float(lo)] * 8 + [float(lo + 1)] * 8))
    assert blpg.backend_of(mine).n_host_staged >= 2
    log("subgroup service ok")

# all_to_all with equal splits: rank r sends value 100*r + d to rank d
src = torch.stack([torch.full((3,), float(100 * rank + d), device=dev) for d in range(world)]).view(-1)
dst = torch.empty_like(src)
dist.all_to_all_single(dst, src)
assert torch.equal(dst.view(world, 3)[:, 0].cpu(), torch.tensor([float(100 * r + rank) for r in range(world)]))
for bad in (lambda: dist.all_reduce(torch.ones(4, dtype=torch.int32, device=dev), op=dist.ReduceOp.BAND),
            lambda: dist.all_reduce(torch.ones(4, dtype=torch.int64, device=dev)),
            lambda: dist.send(torch.ones(4, device=dev), rank)):
    try:
        bad()
        raise SystemExit("expected an error")
    except (RuntimeError, ValueError):
        pass
t = torch.ones(16, device=dev)
dist.all_reduce(t)
assert torch.all(t == world)
log("error paths ok")

# ---- a wait that runs out: status, no trap, link usable again after reset ----------------------
host_barrier()
torch.cuda.synchronize()
# (not with arenas bound to a multicast object: failure cases run with plain peer memory only)
run_timeout_case = not info["multicast"]
if run_timeout_case:
    bl.set_wait_timeout_ms(200)
if run_timeout_case and rank == 0 and world >= 2:
    t = torch.zeros(64, device=dev)
    bl.recv_into(t, 1)  # rank 1 never sends this message
    torch.cuda.synchronize()
    st = bl.status()
    assert st["code"] == 1 and st["from_rank"] == 1, st
    try:
        bl.allreduce_into(t, t)
        raise SystemExit("expected the poisoned link to refuse")
    except RuntimeError:
        pass
host_barrier()
if run_timeout_case:
    bl.reset()
    bl.set_wait_timeout_ms(2000)
host_barrier()
t = torch.ones(64, device=dev)
dist.all_reduce(t)
assert torch.all(t == world) and bl.status()["code"] == 0
log("bounded wait + reset ok")

# ---- latency (device-timed, max over ranks is taken by the caller's log) -------------------------
for nbytes in (10240, 65536, 262144, 1 << 20):
    t = torch.zeros(nbytes // 2, dtype=torch.bfloat16, device=dev)
    for _ in range(10):
        dist.all_reduce(t)
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(50):
        bl.allreduce_into(t, t)
    e1.record()
    torch.cuda.synchronize()
    us = torch.tensor([e0.elapsed_time(e1) / 50 * 1e3])
    dist.all_reduce(us, op=dist.ReduceOp.MAX)
    log("all_reduce %7d B: %.1f us (direct call, max over ranks)" % (nbytes, us.item()))

host_barrier()
dist.destroy_process_group()
bl.shutdown()
print("[pg] rank %d done" % rank, flush=True)
