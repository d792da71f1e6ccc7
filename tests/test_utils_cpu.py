# SPDX-License-Identifier: MIT
"""Observability helpers on CPU: the op tracer restores what it patches, the
clock sampler parses nvidia-smi rows and flags throttle reasons."""
import torch

from barlink_sm86_b200 import ops
from barlink_sm86_b200.utils import ClockSampler, OpTrace, link_stats, max_over_ranks


def test_op_trace_records_and_restores():
    before = ops.linear
    with OpTrace(capacity=4) as t:
        x, w = torch.randn(4, 8), torch.randn(6, 8)
        for _ in range(3):
            ops.linear(x, w)
        ops.rmsnorm(x, torch.ones(8), 1e-6)
        ops.silu_mul(torch.randn(2, 8))
    assert ops.linear is before
    agg = t.summary()
    assert len(t.records) == 4                      # ring buffer keeps the newest records
    assert agg["linear"]["count"] == 2 and agg["rmsnorm"]["count"] == 1 and agg["silu_mul"]["count"] == 1
    assert agg["linear"]["bytes"] == 2 * (4 * 8 + 6 * 8) * 4
    assert "linear" in t.table()


def test_clock_sampler_parse():
    text = ("0, 1905, 1965, 812.33, 0x0000000000000004, Not Active, Not Active, Not Active, Active\n"
            "0, 1410, 1965, 990.10, 0x0000000000000004, Not Active, Active, Not Active, Active\n"
            "garbage line\n")
    r = ClockSampler.parse(text)
    assert r["samples"] == 2 and r["sm_max_mhz"] == 1965.0 and r["sm_mhz"] == (1905 + 1410) / 2
    assert r["reasons"] == ["hw_thermal_slowdown", "sw_power_cap"]


def test_helpers_without_a_link():
    assert isinstance(link_stats(), dict)
    assert max_over_ranks(3.5) == 3.5
