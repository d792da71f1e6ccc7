# SPDX-License-Identifier: MIT
"""The N-rank collective protocols on ONE GPU: four ranks (BL_TEST_WORLD, up
to 8) share device 0 and every collective runs as one cooperative kernel over
all ranks' data, which is how protocols that wait on peers may be exercised
without several GPUs."""
import os

import pytest
import torch

from conftest import rel_l2

pytestmark = pytest.mark.gpu

WORLD = int(os.environ.get("BL_TEST_WORLD", "4"))


@pytest.fixture(scope="module")
def link(ext):
    ext.shutdown()
    ext.init([0] * WORLD, 256)
    yield ext
    ext.shutdown()


def _ints(n, dtype, seed):
    g = torch.Generator(device="cuda").manual_seed(seed)
    return torch.randint(-3, 4, (n,), generator=g, device="cuda").to(dtype)


def test_info_and_verify(link):
    info = link.info()
    assert info["world"] == WORLD and not info["peer_mode"]
    assert link.verify() == 0
    assert link.verify() == 0


DTYPES = [torch.float32, torch.bfloat16, torch.float16, torch.float64, torch.uint8,
          torch.float8_e4m3fn, torch.float8_e5m2]


@pytest.mark.parametrize("dtype", DTYPES)
@pytest.mark.parametrize("algo", ["oneshot", "twoshot"])
def test_allreduce_exact_small_integers(link, dtype, algo):
    n = 4096 + 16
    ins = []
    for r in range(WORLD):
        if dtype == torch.uint8:
            g = torch.Generator(device="cuda").manual_seed(r)
            ins.append(torch.randint(0, 256, (n,), generator=g, device="cuda", dtype=torch.uint8))
        else:
            ins.append(_ints(n, torch.float32, r).to(dtype))
    outs = [torch.empty_like(t) for t in ins]
    link.sp_collective("allreduce", ins, outs, algo=algo)
    torch.cuda.synchronize()
    if dtype == torch.uint8:
        want = sum(t.to(torch.int32) for t in ins).remainder(256).to(torch.uint8)
    else:
        want = sum(t.float() for t in ins).to(dtype)
    for o in outs:
        assert torch.equal(o.view(torch.uint8), want.view(torch.uint8))


@pytest.mark.parametrize("nbytes", [16, 1024, 100 * 1024, 2 * 1024 * 1024 + 48])
def test_allreduce_sizes_and_reuse(link, nbytes):
    n = nbytes // 2
    for it in range(4):  # back to back: inbox rotation and epoch counters
        ins = [torch.randn(n, device="cuda", generator=torch.Generator("cuda").manual_seed(10 * it + r))
               .to(torch.bfloat16) for r in range(WORLD)]
        outs = [torch.empty_like(t) for t in ins]
        link.sp_collective("allreduce", ins, outs)
        want = sum(t.float() for t in ins).to(torch.bfloat16)
        for o in outs:
            assert torch.equal(o, want), (nbytes, it)
    assert link.status()["code"] == 0


def test_allreduce_in_place_pool_tensors(link):
    ts = [link.empty(4096 * 4, r, torch.float32) for r in range(WORLD)]
    for r, t in enumerate(ts):
        t.fill_(float(r + 1))
    link.allreduce_(ts)
    torch.cuda.synchronize()
    for t in ts:
        assert torch.all(t == float(sum(range(1, WORLD + 1))))
    for r, t in enumerate(ts):
        link.free_(t, r)


def test_allgather_reduce_scatter_broadcast(link):
    n = 3000 * 8
    ins = [_ints(n, torch.bfloat16, 100 + r) for r in range(WORLD)]
    outs = [torch.empty(WORLD * n, dtype=torch.bfloat16, device="cuda") for _ in range(WORLD)]
    link.sp_collective("allgather", ins, outs)
    want = torch.cat(ins)
    for o in outs:
        assert torch.equal(o, want)
    big = [_ints(WORLD * n, torch.float32, 200 + r) for r in range(WORLD)]
    outs = [torch.empty(n, dtype=torch.float32, device="cuda") for _ in range(WORLD)]
    link.sp_collective("reduce_scatter", big, outs)
    tot = sum(big)
    for r, o in enumerate(outs):
        assert torch.equal(o, tot[r * n:(r + 1) * n])
    for root in (0, WORLD - 1):
        bufs = [_ints(n, torch.float32, 300 + r) for r in range(WORLD)]
        src = bufs[root].clone()
        link.sp_collective("broadcast", bufs, bufs, root=root)
        for b in bufs:
            assert torch.equal(b, src)
    link.sp_collective("barrier")
    torch.cuda.synchronize()
    assert link.status()["code"] == 0


@pytest.mark.parametrize("rows,hidden", [(1, 3584), (8, 3584), (64, 3584), (3, 5120), (5, 512)])
def test_allreduce_rmsnorm_matches_unfused(link, rows, hidden):
    from barlink_sm86_b200.ops import reference as ref
    g = torch.Generator(device="cuda").manual_seed(rows * 7 + hidden)
    xs = [torch.randn(rows, hidden, device="cuda", generator=g).to(torch.bfloat16) for _ in range(WORLD)]
    res = torch.randn(rows, hidden, device="cuda", generator=g).to(torch.bfloat16)
    gamma = (1 + 0.1 * torch.randn(hidden, device="cuda", generator=g)).to(torch.bfloat16)
    normed = [torch.empty_like(x) for x in xs]
    res_out = [torch.empty_like(x) for x in xs]
    link.sp_collective("allreduce_rmsnorm", xs, normed, [res.clone() for _ in xs], res_out,
                       [gamma.clone() for _ in xs], eps=1e-6)
    want_n, want_r = ref.allreduce_rmsnorm(xs, res, gamma, 1e-6)
    for n_, r_ in zip(normed, res_out):
        assert torch.equal(r_, want_r)
        assert rel_l2(n_, want_n) < 5e-3
    # every rank holds the same bits
    for n_ in normed[1:]:
        assert torch.equal(n_, normed[0])


def test_sendrecv_pairs_and_reuse(link):
    for it in range(5):
        a = torch.arange(1024 * (it + 1), device="cuda", dtype=torch.float32) + it
        b = torch.empty_like(a)
        link.sp_sendrecv(0, 1, a, b)
        link.sp_sendrecv(1, 0, b, a.clone())
        assert torch.equal(a, b)
    x = torch.randint(0, 255, (4096,), device="cuda", dtype=torch.uint8)
    y = torch.empty_like(x)
    link.sp_sendrecv(3, 2, x, y)
    assert torch.equal(x, y)
    assert link.status()["code"] == 0


def test_argument_errors_come_before_traffic(link):
    a = torch.zeros(10, device="cuda")  # 40 bytes: not a multiple of 16
    with pytest.raises(RuntimeError):
        link.sp_collective("allreduce", [a] * WORLD, [a] * WORLD)
    with pytest.raises(RuntimeError):
        link.sp_sendrecv(0, 0, torch.zeros(16, device="cuda"), torch.zeros(16, device="cuda"))
    assert link.status()["code"] == 0
    # the link still works
    ins = [torch.ones(64, device="cuda") for _ in range(WORLD)]
    outs = [torch.empty_like(t) for t in ins]
    link.sp_collective("allreduce", ins, outs)
    assert torch.all(outs[0] == WORLD)
