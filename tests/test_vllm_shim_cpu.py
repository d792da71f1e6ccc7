# SPDX-License-Identifier: MIT
"""The vLLM hook against stand-ins for the vLLM objects it patches (no GPU,
no engine start)."""
import importlib
import os
import sys
import types

import pytest


@pytest.fixture
def fake_vllm(monkeypatch):
    """Minimal module tree with the attributes the hook touches."""
    mods = {}

    def mk(name):
        m = types.ModuleType(name)
        mods[name] = m
        monkeypatch.setitem(sys.modules, name, m)
        return m

    mk("vllm")
    mk("vllm.platforms")
    cuda = mk("vllm.platforms.cuda")
    cuda.CudaPlatformBase = type("CudaPlatformBase", (), {"dist_backend": "nccl"})
    mk("vllm.distributed")
    mk("vllm.distributed.device_communicators")
    cc = mk("vllm.distributed.device_communicators.cuda_communicator")

    class CudaCommunicator:
        world_size = 2

        def all_reduce(self, x):
            return ("stock", x)

    cc.CudaCommunicator = CudaCommunicator
    sys.modules["vllm.distributed.device_communicators"].cuda_communicator = cc
    for k in ("BL_SHIM_OFF", "BL_SHIM_STEPS", "VLLM_DISABLE_PYNCCL", "VLLM_ALLREDUCE_USE_SYMM_MEM"):
        monkeypatch.delenv(k, raising=False)
    return mods


def _fresh_shim():
    sys.modules.pop("vllm_barlink", None)
    return importlib.import_module("vllm_barlink")


def test_backend_string_rewrite():
    shim = _fresh_shim()
    assert shim.rewrite_backend("cpu:gloo,cuda:nccl") == "cpu:gloo,cuda:barlink"
    assert shim.rewrite_backend("nccl") == "barlink"
    assert shim.rewrite_backend("gloo") == "gloo"
    assert shim.rewrite_backend(None) is None


def test_install_patches_platform_env_and_communicator(fake_vllm, monkeypatch):
    import torch.distributed as dist
    monkeypatch.setattr(dist, "init_process_group", lambda *a, **k: ("called", a, k))
    monkeypatch.setattr(dist, "is_backend_available", lambda b: b in ("gloo", "nccl"))
    shim = _fresh_shim()
    assert fake_vllm["vllm.platforms.cuda"].CudaPlatformBase.dist_backend == "barlink"
    assert os.environ["VLLM_DISABLE_PYNCCL"] == "1"
    cc = fake_vllm["vllm.distributed.device_communicators.cuda_communicator"].CudaCommunicator
    assert getattr(cc.all_reduce, "_barlink_wrapped", False)
    # CPU tensors keep vLLM's own path
    import torch
    assert cc().all_reduce(torch.ones(4))[0] == "stock"
    # the wrapped init rewrites the backend and registers lazily
    r = dist.init_process_group(backend="cpu:gloo,cuda:nccl", rank=0, world_size=1)
    assert r[2]["backend"] == "cpu:gloo,cuda:barlink"
    assert shim._registered
    r = dist.init_process_group("gloo")
    assert r[1][0] == "gloo"


def test_shim_off_and_step_selection(fake_vllm, monkeypatch):
    import torch.distributed as dist
    sentinel = lambda *a, **k: "orig"  # noqa: E731
    monkeypatch.setattr(dist, "init_process_group", sentinel)
    monkeypatch.setenv("BL_SHIM_OFF", "1")
    _fresh_shim()
    assert dist.init_process_group is sentinel
    assert fake_vllm["vllm.platforms.cuda"].CudaPlatformBase.dist_backend == "nccl"
    monkeypatch.delenv("BL_SHIM_OFF")
    monkeypatch.setenv("BL_SHIM_STEPS", "3")
    _fresh_shim()
    assert dist.init_process_group is sentinel  # steps 1, 2 off
    assert fake_vllm["vllm.platforms.cuda"].CudaPlatformBase.dist_backend == "barlink"


def test_entry_trampoline_installs_the_hook_in_the_child(tmp_path):
    """`entry.py script.py` must leave torch.distributed.init_process_group wrapped in the
    re-executed interpreter (and unwrapped with BL_SHIM_OFF=1)."""
    import subprocess

    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    script = tmp_path / "probe.py"
    script.write_text(
        "import os, torch.distributed as dist\n"
        "print('WRAPPED=%d SHIM=%s' % (int(getattr(dist.init_process_group, '_barlink_wrapped', False)),"
        " os.environ.get('BL_SHIM', '')))\n")
    env = {k: v for k, v in os.environ.items() if not k.startswith("BL_SHIM") and k != "PYTHONPATH"}
    entry = os.path.join(root, "vllm_barlink", "entry.py")
    out = subprocess.run([sys.executable, entry, str(script)], env=env, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr
    assert "WRAPPED=1 SHIM=1" in out.stdout, out.stdout + out.stderr
    env["BL_SHIM_OFF"] = "1"
    out = subprocess.run([sys.executable, entry, str(script)], env=env, capture_output=True, text=True,
                         timeout=300)
    assert out.returncode == 0, out.stderr
    assert "WRAPPED=0" in out.stdout, out.stdout + out.stderr
