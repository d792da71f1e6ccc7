# SPDX-License-Identifier: MIT
"""Measurement and observability helpers: device timing, GPU clock sampling,
an op-level tracer with NVTX ranges, and the link's counter block.

The reference has no built-in tracer; it uses ad-hoc torch.profiler scripts,
CUDA-event pairs around hooked all-reduces and per-run stats files
(demos/qwen_tp/qwen38_int8/profile_decode.py:24-44, worker.py:157-179,
:648-661).  These helpers are the library form of that."""
from .checkpoint import SafetensorsSource, config_from_hf, save_qwen2_safetensors
from .clocks import ClockSampler
from .timing import cuda_time_us, flush_l2, max_over_ranks
from .trace import OpTrace, link_stats

__all__ = ["SafetensorsSource", "config_from_hf", "save_qwen2_safetensors", "ClockSampler", "cuda_time_us", "flush_l2", "max_over_ranks", "OpTrace", "link_stats"]
