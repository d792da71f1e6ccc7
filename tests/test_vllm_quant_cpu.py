# SPDX-License-Identifier: MIT
"""The vLLM quantization method "barlink_w8a16" against the installed vLLM on
CPU: registration, post-load quantisation of a layer, and the linear against
the fp32 product (the CPU statement of the W8A16 op runs underneath)."""
import subprocess
import sys
import os

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

SCRIPT = r"""
import sys, torch
sys.path.insert(0, %r)
import vllm_barlink.quant as q
assert q.register() == "barlink_w8a16" and q.register() == "barlink_w8a16"   # idempotent
from vllm.model_executor.layers.quantization import get_quantization_config
cfg = get_quantization_config("barlink_w8a16").from_config({})
assert cfg.get_name() == "barlink_w8a16" and cfg.get_min_capability() == 100
assert cfg.get_supported_act_dtypes() == [torch.bfloat16] and cfg.get_config_filenames() == []
assert cfg.get_quant_method(torch.nn.Embedding(4, 4), "embed") is None
m = q.register.method_cls()
layer = torch.nn.Module()
g = torch.Generator().manual_seed(0)
w = torch.randn(96, 64, generator=g) * 0.05
layer.weight = torch.nn.Parameter(w.clone().to(torch.bfloat16), requires_grad=False)
m.process_weights_after_loading(layer)
assert layer.bl_wq.dtype == torch.int8 and layer.bl_wq.shape == (96, 64) and layer.bl_scale.shape == (96,)
assert layer.weight.numel() == 0                       # the bf16 copy is gone
x = torch.randn(2, 5, 64, generator=g).to(torch.bfloat16)
b = torch.randn(96, generator=g).to(torch.bfloat16)
y = m.apply(layer, x, b)
ref = x.float() @ w.t() + b.float()
err = ((y.float() - ref).norm() / ref.norm()).item()
assert y.shape == (2, 5, 96) and err < 1e-2, err
# the op is traceable: fake tensors give the output shape without running it
from torch._subclasses.fake_tensor import FakeTensorMode
with FakeTensorMode():
    fy = torch.ops.barlink.w8a16_linear(torch.empty(3, 64, dtype=torch.bfloat16), torch.empty(96, 64, dtype=torch.int8),
                                         torch.empty(96, dtype=torch.bfloat16), None)
assert tuple(fy.shape) == (3, 96)
print("QUANT OK %%.4f" %% err)
"""


def test_barlink_w8a16_method_registers_and_matches_fp32():
    try:
        import vllm  # noqa: F401
    except Exception:
        pytest.skip("vLLM is not importable here")
    # own interpreter: importing vLLM's model executor is heavy and leaves global state behind
    p = subprocess.run([sys.executable, "-c", SCRIPT % ROOT], capture_output=True, text=True, timeout=600)
    assert p.returncode == 0 and "QUANT OK" in p.stdout, p.stdout[-1500:] + p.stderr[-3000:]


def test_quantization_config_pickles_by_reference():
    """vLLM starts its engine and worker processes with `spawn` once CUDA is initialised and pickles the
    configuration for them: the method's classes must travel by reference (classes defined inside a function
    would be pickled by value, together with `torch.ops`, which cannot be)."""
    import pickle

    pytest.importorskip("vllm")
    cloudpickle = pytest.importorskip("cloudpickle")
    from vllm_barlink import quant

    quant.register()
    cfg = quant.register.config_cls()
    for obj in (cfg, quant.register.config_cls, quant.register.method_cls()):
        blob = cloudpickle.dumps(obj)
        assert len(blob) < 4096          # a reference, not the class body
        back = pickle.loads(blob)
        assert (back if isinstance(back, type) else type(back)).__module__ == "vllm_barlink._quant_classes"
