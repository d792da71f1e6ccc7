# SPDX-License-Identifier: MIT
"""Host-side arithmetic of the link core, without a GPU: arena layout, the
symmetric allocator, the all-reduce algorithm table and the k-split choice."""
import pytest

import barlink_sm86_b200 as bl

C = bl.load_extension()
MB = 1 << 20


@pytest.mark.parametrize("world", [2, 3, 4, 8])
@pytest.mark.parametrize("pool_mb", [64, 256, 1024, 4096])
def test_layout_zones_are_ordered_aligned_and_disjoint(world, pool_mb):
    L = C.layout_of(pool_mb * MB, world)
    assert 0 < L["user_bytes"] == L["stage_off"]
    stage_end = L["stage_off"] + 4 * world * L["stage_slice"]
    lamport_end = L["lamport_off"] + 3 * world * L["lamport_slice"]
    p2p_end = L["p2p_off"] + world * L["p2p_slice"]
    assert stage_end <= L["lamport_off"] and lamport_end <= L["p2p_off"] and p2p_end <= L["sig_off"] < L["pool_bytes"]
    for k in ("stage_off", "lamport_off", "p2p_off"):
        assert L[k] % 65536 == 0
    for k in ("stage_slice", "lamport_slice", "p2p_slice"):
        assert L[k] % 4096 == 0 and L[k] > 0
    assert L["user_bytes"] >= L["pool_bytes"] // 2      # callers keep most of the arena
    assert L["lamport_slice"] <= MB                      # the one-shot inbox never outgrows 1 MiB


def test_allocator_first_fit_reuse_and_errors():
    user = 8 * MB
    r = C.arena_replay(user, [("alloc", 100), ("alloc", 4096), ("alloc", 1)])
    assert r == [0, 256, 256 + 4096]                       # 16-byte rounding, 256-byte alignment
    # a freed block is reused; a large request is 2 MiB aligned
    r = C.arena_replay(user, [("alloc", 1000), ("alloc", 1000), ("free", 0, 1000), ("alloc", 500),
                              ("alloc", 3 * MB), ("alloc", 4 * MB)])
    assert r[3] == 0 and r[4] == 2 * MB and r[5] == -1     # 2 + 3 MiB used: 4 MiB no longer fits in 8
    # double free and out-of-range free are refused
    r = C.arena_replay(user, [("alloc", 4096), ("free", 0, 4096), ("free", 0, 4096), ("free", 1 << 22, 16)])
    assert r[1:] == [1, 0, 0]
    # neighbours coalesce: after freeing both halves the whole range is one block again
    r = C.arena_replay(user, [("alloc", MB), ("alloc", MB), ("free", 0, MB), ("free", MB, MB), ("alloc", 2 * MB)])
    assert r[-1] == 0


def test_allreduce_algorithm_table():
    assert C.algo_for(4096, 2) == "oneshot" and C.algo_for(MB, 2) == "oneshot" and C.algo_for(4 * MB, 2) == "twoshot"
    assert C.algo_for(512 << 10, 8) == "oneshot" and C.algo_for(MB, 8) == "twoshot"
    # types the one-shot kernel cannot flag (every bit pattern is data) go two-shot
    assert C.algo_for(4096, 8, "fp64") == "twoshot" and C.algo_for(4096, 8, "u8") == "twoshot"
    # NVLS only where a multicast object exists, only for large bf16/fp16/fp32 messages
    assert C.algo_for(4 * MB, 8, "bf16", True) == "nvls" and C.algo_for(4 * MB, 8, "bf16", False) == "twoshot"
    assert C.algo_for(4 * MB, 8, "u8", True) == "twoshot"
    # a forced algorithm that cannot run falls back instead of failing
    assert C.algo_for(64 * MB, 8, "bf16", False, 1 << 30, "oneshot") == "twoshot"
    assert C.algo_for(4096, 8, "bf16", False, 1 << 30, "nvls") == "twoshot"


@pytest.mark.parametrize("tiles,kblocks", [(1, 1), (6, 56), (37, 56), (28, 8), (149, 56), (296, 56), (1188, 56)])
def test_k_split_choice(tiles, kblocks):
    s = C.pick_splits(tiles, kblocks)
    assert 1 <= s <= kblocks
    per = -(-kblocks // s)
    assert -(-kblocks // per) == s                          # every split owns at least one k-block
    if tiles >= 148:
        assert s == 1                                       # enough tiles: no split
    if tiles * kblocks >= 148 and tiles < 74:
        assert s > 1                                        # few tiles with a long k: split


@pytest.mark.parametrize("n,k,tokens", [(768, 3584, 64), (3584, 512, 64), (4736, 3584, 64), (3584, 2368, 64),
                                        (37888, 3584, 64), (256, 128, 1), (19008, 3584, 8), (128, 64, 16)])
def test_decode_linear_cluster_choice(n, k, tokens):
    """Cluster size of the decode linears (host arithmetic, no GPU needed): between 1 and 8, never
    more CTAs than k-blocks, at least two k-blocks per CTA when the product is split, a forced size
    is honoured up to those limits, and a shape with two full waves of tiles is not split at all
    (149 tiles on 148 SMs may be: two laps of half the k-blocks beat one lap plus one tile)."""
    kblocks = -(-k // 64)
    auto = C.dlin_cluster(n, k, tokens, 0)
    assert 1 <= auto <= 8 and auto <= max(1, kblocks)
    if auto > 1:
        assert kblocks // auto >= 2
    if -(-n // 128) >= 2 * 148:
        assert auto == 1
    for want in (1, 2, 4, 8):
        got = C.dlin_cluster(n, k, tokens, want)
        assert 1 <= got <= min(want, max(1, kblocks))
