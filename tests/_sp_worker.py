# SPDX-License-Identifier: MIT
"""Single-process mode on N real GPUs (started by test_pg_gpu.py): one process
drives every GPU, `bl.init(devices, pool_mb)`, pool tensors, copy_ between
arenas, allreduce_ and the list collectives.  The reference's unit tests of
this mode: torch_ext/tests/test_basic.py:29-112, test_dtypes.py:21-92,
test_chunked.py:17-67."""
import os
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import barlink_sm86_b200 as bl  # noqa: E402

n = int(sys.argv[1])
devs = list(range(n))
bl.init(devs, 256)
info = bl.info()
assert info["world"] == n and not info["peer_mode"], info
assert bl.verify() == 0

# pool tensors, copy_ from every arena to the next, byte-exact
size = 4 << 20
srcs = [bl.empty(size, r, torch.uint8) for r in devs]
dsts = [bl.empty(size, r, torch.uint8) for r in devs]
for r, s in enumerate(srcs):
    g = torch.Generator(device="cuda:%d" % r).manual_seed(r)
    s.copy_(torch.randint(0, 256, (size,), generator=g, device="cuda:%d" % r, dtype=torch.uint8))
for r in devs:
    bl.copy_(dsts[(r + 1) % n], srcs[r])
for r in devs:
    torch.cuda.synchronize(r)
for r in devs:
    assert torch.equal(dsts[(r + 1) % n].cpu(), srcs[r].cpu()), "copy_ %d -> %d" % (r, (r + 1) % n)

# allreduce_ on pool tensors, every dtype, values whose sum is exact
for dt in (torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.uint8):
    ts = [bl.empty(65536 * 4, r, dt) for r in devs]
    vals = []
    for r, t in enumerate(ts):
        g = torch.Generator(device="cuda:%d" % r).manual_seed(100 + r)
        v = torch.randint(0, 4, (t.numel(),), generator=g, device="cuda:%d" % r)
        t.copy_(v.to(dt))
        vals.append(v.cpu())
    bl.allreduce_(ts)
    for r in devs:
        torch.cuda.synchronize(r)
    want = sum(vals)
    want = want.remainder(256).to(torch.uint8) if dt == torch.uint8 else want.to(dt)
    for t in ts:
        assert torch.equal(t.cpu(), want), dt
    for r, t in enumerate(ts):
        bl.free_(t, r)

# chunked helpers on a tensor larger than one call's limit
big = max(info["max_chunk"] + (1 << 20) + 16, 8 << 20)
a = [bl.empty(big, r, torch.uint8) for r in devs]
for r, t in enumerate(a):
    t.fill_(r + 1)
bl.allreduce_large(a, chunk_bytes=(4 << 20) + 16)
for r in devs:
    torch.cuda.synchronize(r)
assert all(int(t[::4099].max()) == int(t[::4099].min()) == sum(range(1, n + 1)) % 256 for t in a)
b = bl.empty(big, 0, torch.uint8)
bl.copy_large(b, a[n - 1], chunk_bytes=(4 << 20) + 16)
torch.cuda.synchronize(0)
assert torch.equal(b[:4096].cpu(), a[n - 1][:4096].cpu())

# list collectives on ordinary (non-pool) tensors, one per GPU
xs = [torch.full((3000 * 8,), float(r + 1), device="cuda:%d" % r, dtype=torch.bfloat16) for r in devs]
outs = [torch.empty_like(x) for x in xs]
C = bl.load_extension()
for algo in ("oneshot", "twoshot"):
    C.sp_collective("allreduce", xs, outs, algo=algo)
    for r in devs:
        torch.cuda.synchronize(r)
    assert all(torch.all(o == float(sum(range(1, n + 1)))) for o in outs), algo
gath = [torch.empty(n * x.numel(), device=x.device, dtype=x.dtype) for x in xs]
C.sp_collective("allgather", xs, gath)
for r in devs:
    torch.cuda.synchronize(r)
want = torch.cat([x.cpu() for x in xs])
assert all(torch.equal(g.cpu(), want) for g in gath)
assert bl.status()["code"] == 0
bl.shutdown()
print("single-process mode on %d GPUs ok" % n)
