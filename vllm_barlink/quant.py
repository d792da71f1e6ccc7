# SPDX-License-Identifier: MIT
"""vLLM quantization method "barlink_w8a16": every linear layer keeps bf16
activations and holds int8 weights with one bf16 scale per output channel, and
its matrix product is this library's tcgen05 W8A16 kernel (int8 widened to
bf16 inside the main loop).

The layer first receives ordinary bf16 weights, exactly as an unquantised
layer would (so any checkpoint, vLLM's dummy weights and the merged QKV /
gate-up loaders work unchanged); `process_weights_after_loading` then
quantises the local shard symmetric per output channel and drops the bf16
copy.  The reference reaches the same end state by unpacking an INT8
checkpoint in its own worker (demos/qwen_tp/qwen38_int8/worker.py:97-150);
inside vLLM it relied on vLLM's own kernels.

    import vllm_barlink.quant; vllm_barlink.quant.register()
    LLM(model=..., quantization="barlink_w8a16")

Spawned vLLM workers register through the entry hook: step 6 of
`BL_SHIM_STEPS` (opt-in), e.g. BL_SHIM_STEPS=1,2,3,4,6.
"""
import os
import sys

import torch

NAME = "barlink_w8a16"
_registered = False
_op_defined = False


def _ops():
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from barlink_sm86_b200 import ops

    return ops


def _define_op():
    """One traceable op, so that torch.compile / CUDA-graph capture of the
    model sees an opaque call with a known output shape."""
    global _op_defined
    if _op_defined:
        return
    _op_defined = True

    @torch.library.custom_op("barlink::w8a16_linear", mutates_args=())
    def w8a16_linear(x: torch.Tensor, wq: torch.Tensor, scale: torch.Tensor, bias: torch.Tensor | None) -> torch.Tensor:
        x2 = x.reshape(-1, x.shape[-1])
        if x2.is_cuda and not x2.is_contiguous():
            x2 = x2.contiguous()
        y = _ops().w8a16_linear(x2, wq, scale, bias)
        return y.reshape(*x.shape[:-1], wq.shape[0])

    @w8a16_linear.register_fake
    def _(x, wq, scale, bias):
        return x.new_empty(*x.shape[:-1], wq.shape[0])


def quantize_channelwise(w):
    """[n, k] weight -> (int8 [n, k], bf16 scale [n]), symmetric per output channel."""
    wf = w.float()
    scale = (wf.abs().amax(1).clamp_min(1e-12) / 127.0).to(torch.bfloat16)
    wq = torch.round(wf / scale.float()[:, None]).clamp(-127, 127).to(torch.int8)
    return wq.contiguous(), scale.contiguous()


def register():
    """Make quantization="barlink_w8a16" known to vLLM (idempotent).  The classes live at the top level of
    `vllm_barlink._quant_classes` (imported here, because it needs vLLM) so that vLLM can pickle a config that
    carries them by reference when it starts its engine and worker processes with `spawn`."""
    global _registered
    if _registered:
        return NAME
    _define_op()
    from . import _quant_classes as qc

    BarlinkW8A16Config, BarlinkW8A16LinearMethod = qc.BarlinkW8A16Config, qc.BarlinkW8A16LinearMethod
    register.config_cls = BarlinkW8A16Config
    register.method_cls = BarlinkW8A16LinearMethod
    _registered = True
    return NAME
