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
    """Make quantization="barlink_w8a16" known to vLLM (idempotent)."""
    global _registered
    if _registered:
        return NAME
    from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
    from vllm.model_executor.layers.quantization import register_quantization_config
    from vllm.model_executor.layers.quantization.base_config import QuantizationConfig

    _define_op()

    class BarlinkW8A16LinearMethod(LinearMethodBase):
        def __init__(self):
            self._plain = UnquantizedLinearMethod()

        def create_weights(self, layer, input_size_per_partition, output_partition_sizes, input_size, output_size,
                           params_dtype, **extra_weight_attrs):
            # same parameter as an unquantised layer: every loader keeps working
            self._plain.create_weights(layer, input_size_per_partition, output_partition_sizes, input_size,
                                       output_size, params_dtype, **extra_weight_attrs)

        def process_weights_after_loading(self, layer):
            wq, scale = quantize_channelwise(layer.weight.data)
            layer.register_buffer("bl_wq", wq, persistent=False)
            layer.register_buffer("bl_scale", scale, persistent=False)
            # keep an empty parameter under the old name so that code that only inspects it keeps working
            layer.weight = torch.nn.Parameter(torch.empty(0, dtype=scale.dtype, device=wq.device), requires_grad=False)

        def apply(self, layer, x, bias=None):
            if x.dtype != torch.bfloat16 and x.is_cuda:
                return torch.ops.barlink.w8a16_linear(x.to(torch.bfloat16), layer.bl_wq, layer.bl_scale,
                                                      None if bias is None else bias.to(torch.bfloat16)).to(x.dtype)
            return torch.ops.barlink.w8a16_linear(x, layer.bl_wq, layer.bl_scale, bias)

    @register_quantization_config(NAME)
    class BarlinkW8A16Config(QuantizationConfig):
        def get_name(self):
            return NAME

        def get_supported_act_dtypes(self):
            return [torch.bfloat16]

        @classmethod
        def get_min_capability(cls):
            return 100  # the kernel is written for sm_100a

        @staticmethod
        def get_config_filenames():
            return []  # nothing is read from the checkpoint: weights are quantised after loading

        @classmethod
        def from_config(cls, config):
            return cls()

        def get_quant_method(self, layer, prefix):
            if isinstance(layer, LinearBase):
                return BarlinkW8A16LinearMethod()
            return None  # embeddings, the LM head's vocab embedding and attention stay as they are

    register.config_cls = BarlinkW8A16Config
    register.method_cls = BarlinkW8A16LinearMethod
    _registered = True
    return NAME
