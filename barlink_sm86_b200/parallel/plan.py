# SPDX-License-Identifier: MIT
"""Deterministic sharding rules for tensor parallelism.

Counterpart of the reference's shard rules (demos/qwen_tp/qwen38_int8/
worker.py:248-279: column shards narrow the output dim, row shards the input
dim, fused QKV is cut per head group), extended to TP up to 8 with fewer KV
heads than ranks: a KV head is then replicated on `tp / nkv` ranks and its
query heads are dealt out among them, padded with empty slots so that every
rank has the same shapes (an empty slot has zero weights and contributes
nothing to the row-parallel sum).
"""
from dataclasses import dataclass
from typing import List

import torch


@dataclass
class HeadPlan:
    q_heads: List[int]    # global query head per local slot, -1 = empty slot
    kv_heads: List[int]   # global KV head per local slot
    @property
    def nq(self):
        return len(self.q_heads)

    @property
    def nkv(self):
        return len(self.kv_heads)


def head_plan(nq: int, nkv: int, tp: int, rank: int) -> HeadPlan:
    if nq % nkv:
        raise ValueError("query heads (%d) must be a multiple of KV heads (%d)" % (nq, nkv))
    g = nq // nkv
    if nkv % tp == 0:
        per = nkv // tp
        kv = list(range(rank * per, (rank + 1) * per))
        q = [h * g + i for h in kv for i in range(g)]
        return HeadPlan(q, kv)
    if tp % nkv == 0:
        rep = tp // nkv
        j, sub = divmod(rank, rep)
        per = -(-g // rep)
        q = [(j * g + sub * per + i) if sub * per + i < g else -1 for i in range(per)]
        return HeadPlan(q, [j])
    raise ValueError("tp=%d must divide or be a multiple of the %d KV heads" % (tp, nkv))


def shard_rows(w: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Column-parallel shard: rows (output features) [rank*n/tp, (rank+1)*n/tp)."""
    n = w.shape[0]
    if n % tp:
        raise ValueError("cannot split %d output features over %d ranks" % (n, tp))
    per = n // tp
    return w[rank * per:(rank + 1) * per].contiguous()


def shard_cols(w: torch.Tensor, tp: int, rank: int) -> torch.Tensor:
    """Row-parallel shard: columns (input features) [rank*k/tp, (rank+1)*k/tp)."""
    k = w.shape[1]
    if k % tp:
        raise ValueError("cannot split %d input features over %d ranks" % (k, tp))
    per = k // tp
    return w[:, rank * per:(rank + 1) * per].contiguous()


def interleave_gate_up(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """Rows (gate_0, up_0, gate_1, up_1, ...): the layout whose GEMM epilogue
    can apply SiLU(gate)*up on adjacent accumulator rows/columns."""
    n, k = gate.shape
    out = torch.empty(2 * n, k, dtype=gate.dtype, device=gate.device)
    out[0::2] = gate
    out[1::2] = up
    return out


def gather_heads(w: torch.Tensor, heads: List[int], hd: int) -> torch.Tensor:
    """Rows of a [n_heads*hd, k] projection for the listed heads; -1 gives zeros."""
    k = w.shape[1:]
    out = torch.zeros((len(heads) * hd,) + tuple(k), dtype=w.dtype, device=w.device)
    for i, h in enumerate(heads):
        if h >= 0:
            out[i * hd:(i + 1) * hd] = w[h * hd:(h + 1) * hd]
    return out


def gather_head_cols(w: torch.Tensor, heads: List[int], hd: int) -> torch.Tensor:
    """Columns of a [n, n_heads*hd] projection for the listed heads; -1 gives zeros."""
    out = torch.zeros(w.shape[0], len(heads) * hd, dtype=w.dtype, device=w.device)
    for i, h in enumerate(heads):
        if h >= 0:
            out[:, i * hd:(i + 1) * hd] = w[:, h * hd:(h + 1) * hd]
    return out
