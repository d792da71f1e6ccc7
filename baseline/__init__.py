# SPDX-License-Identifier: MIT
"""Baselines: the reference arm of bench.py and the NCCL(+cuBLAS) restatement
of the reference's decode harness."""
