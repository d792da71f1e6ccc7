# SPDX-License-Identifier: MIT
"""The vLLM-facing classes of the quantization method "barlink_w8a16" (see `vllm_barlink.quant`).
Top-level classes of an importable module: vLLM pickles its configuration when it starts engine and
worker processes with `spawn`, and classes defined inside a function would be pickled by value
together with everything their methods reach (which fails on `torch.ops`).  Importing this module
imports vLLM."""
import torch
from vllm.model_executor.layers.linear import LinearBase, LinearMethodBase, UnquantizedLinearMethod
from vllm.model_executor.layers.quantization import register_quantization_config
from vllm.model_executor.layers.quantization.base_config import QuantizationConfig

from .quant import NAME, _define_op, quantize_channelwise

# a process that gets these classes by unpickling a configuration needs the op as well
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
