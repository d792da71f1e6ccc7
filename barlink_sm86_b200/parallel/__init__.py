# SPDX-License-Identifier: MIT
"""Tensor parallelism over the barlink link.

The reference's only parallelism is Megatron-style TP=2 written into its demo
workers: row-parallel layers finish their partial sums with `dist.all_reduce`
in a forward hook (demos/qwen_tp/qwen38_int8/worker.py:167-183, 248-279),
fused QKV is sharded per head group (:272-279), the lm_head is vocab-parallel
with a gather (:208-241).  Here the same strategy is a small library for
TP = 1, 2, 4, 8: head plans that replicate KV heads when there are fewer of
them than ranks, shard helpers, and a communicator that uses the fused
all-reduce+RMSNorm kernel and the fused GEMM+collective linears on CUDA and
plain c10d collectives (gloo) on CPU.
"""
from .comm import TPComm
from .plan import HeadPlan, head_plan, shard_rows, shard_cols, interleave_gate_up

__all__ = ["TPComm", "HeadPlan", "head_plan", "shard_rows", "shard_cols", "interleave_gate_up"]
