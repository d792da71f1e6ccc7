# SPDX-License-Identifier: MIT
"""Model families served by the library: the Qwen2-style decoder (decode and
prefill, TP 1-8, paged KV, CUDA-graphed step) and the Flux-style MMDiT image
denoiser.  The reference drives HF transformers / diffusers / vLLM models
from its demo workers (demos/qwen_tp, demos/flux2_tp, demos/vllm_bl); these
are the same architectures owned by the library, so that every layer runs the
sm_100a kernels."""
from .mmdit import MMDiTConfig, MMDiTModel, MMDiTWeights, denoise, grid_positions
from .qwen2 import DecodeEngine, PagedKV, Qwen2Config, Qwen2Model, Qwen2Weights, W4Weight, W8Weight, qlinear

__all__ = ["DecodeEngine", "PagedKV", "Qwen2Config", "Qwen2Model", "Qwen2Weights", "W4Weight", "W8Weight", "qlinear",
           "MMDiTConfig", "MMDiTModel", "MMDiTWeights", "denoise", "grid_positions"]
