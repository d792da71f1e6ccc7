# SPDX-License-Identifier: MIT
"""vLLM entry hook: makes vLLM's tensor-parallel collectives run on barlink.

Importing this module (from a `.pth` file, `sitecustomize.py`, or explicitly
before `import vllm`) installs a set of switchable steps, same idea and same
switches as the reference's shim (vllm_barlink/__init__.py:34-142 there):

  1. register the "barlink" c10d backend -- lazily, on first use, because
     importing CUDA code at interpreter start would initialise CUDA in
     vLLM's engine-core process before it forks its workers;
  2. wrap `torch.distributed.init_process_group` (and
     `is_backend_available`) so that a backend string naming nccl for CUDA is
     rewritten to barlink (vLLM asks for "cpu:gloo,cuda:nccl");
  3. default `VLLM_DISABLE_PYNCCL=1`, `VLLM_ALLREDUCE_USE_SYMM_MEM=0` and set
     the CUDA platform's `dist_backend` to "barlink", so that
     `CudaCommunicator` falls through to its torch.distributed path;
  4. give `CudaCommunicator.all_reduce` a direct fast path: a contiguous,
     16-byte-aligned CUDA tensor goes straight to the link's all-reduce kernel
     (one launch, no c10d dispatch); everything else keeps vLLM's own path
     (which, after step 3, ends in the barlink process group);
  5. (opt-in) add `vllm::all_reduce` to the compilation splitting ops so that
     it runs between captured graph pieces.  barlink's collectives are safe to
     capture (their expectations are device counters), so this is only an
     escape hatch;
  6. (opt-in) register the quantization method "barlink_w8a16"
     (`vllm_barlink/quant.py`): linear layers run this library's W8A16 kernel.

`BL_SHIM_STEPS` (default "1,2,3,4") selects steps, `BL_SHIM_OFF=1` disables
the hook, `BL_SHIM_DEBUG=1` logs what it does.
"""
import os
import sys

_DONE = False
_registered = False


def _debug(msg):
    if os.environ.get("BL_SHIM_DEBUG") == "1":
        sys.stderr.write("[vllm_barlink pid %d] %s\n" % (os.getpid(), msg))


def _step(n):
    return str(n) in os.environ.get("BL_SHIM_STEPS", "1,2,3,4").split(",")


def _ensure_registered():
    global _registered
    if _registered:
        return
    _registered = True
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    if root not in sys.path:
        sys.path.insert(0, root)
    from barlink_sm86_b200 import process_group as blpg

    blpg.register()
    _debug("registered the barlink backend")


def rewrite_backend(backend):
    """"cpu:gloo,cuda:nccl" -> "cpu:gloo,cuda:barlink"; "nccl" -> "barlink"."""
    if isinstance(backend, str) and "nccl" in backend:
        return backend.replace("nccl", "barlink")
    return backend


def _fast_all_reduce(orig):
    def all_reduce(self, input_):
        try:
            import torch

            if (getattr(self, "world_size", 1) > 1 and input_.is_cuda and input_.is_contiguous()
                    and input_.data_ptr() % 16 == 0 and (input_.numel() * input_.element_size()) % 16 == 0
                    and input_.dtype in (torch.bfloat16, torch.float16, torch.float32)):
                import barlink_sm86_b200 as bl

                info = bl.info()
                if info.get("initialized") and info.get("peer_mode") and info["world"] == self.world_size \
                        and input_.numel() * input_.element_size() <= info["max_chunk"]:
                    out = torch.empty_like(input_)
                    bl.allreduce_into(out, input_)
                    return out
        except ImportError:
            pass
        return orig(self, input_)

    all_reduce._barlink_wrapped = True
    return all_reduce


def install():
    global _DONE
    if _DONE or os.environ.get("BL_SHIM_OFF") == "1":
        return
    _DONE = True
    _debug("installing steps %s" % os.environ.get("BL_SHIM_STEPS", "1,2,3,4"))

    if _step(1) or _step(2):
        import torch.distributed as dist

        orig_ipg = dist.init_process_group
        if not getattr(orig_ipg, "_barlink_wrapped", False):
            def init_process_group(*args, **kwargs):
                backend = kwargs.get("backend", args[0] if args else None)
                if isinstance(backend, str) and ("nccl" in backend or "barlink" in backend):
                    if _step(1):
                        _ensure_registered()
                    if _step(2):
                        new = rewrite_backend(backend)
                        if "backend" in kwargs:
                            kwargs["backend"] = new
                        else:
                            args = (new,) + tuple(args[1:])
                        _debug("init_process_group backend %r -> %r" % (backend, new))
                return orig_ipg(*args, **kwargs)

            init_process_group._barlink_wrapped = True
            dist.init_process_group = init_process_group

        orig_iba = dist.is_backend_available
        if not getattr(orig_iba, "_barlink_wrapped", False):
            def is_backend_available(backend):
                if backend == "barlink" and _step(1):
                    _ensure_registered()
                return orig_iba(backend)

            is_backend_available._barlink_wrapped = True
            dist.is_backend_available = is_backend_available

    if _step(3):
        os.environ.setdefault("VLLM_DISABLE_PYNCCL", "1")
        os.environ.setdefault("VLLM_ALLREDUCE_USE_SYMM_MEM", "0")
        try:
            from vllm.platforms.cuda import CudaPlatformBase

            CudaPlatformBase.dist_backend = "barlink"
        except Exception as e:  # vLLM absent or laid out differently: the other steps still help
            _debug("platform patch skipped: %s" % e)

    if _step(4):
        try:
            from vllm.distributed.device_communicators import cuda_communicator

            cc = cuda_communicator.CudaCommunicator
            if not getattr(cc.all_reduce, "_barlink_wrapped", False):
                cc.all_reduce = _fast_all_reduce(cc.all_reduce)
            if hasattr(cc, "maybe_init_pynccl_communicator"):
                cc.maybe_init_pynccl_communicator = lambda self: None
        except Exception as e:
            _debug("communicator patch skipped: %s" % e)

    if _step(5):
        try:
            from vllm.config.compilation import CompilationConfig

            orig = CompilationConfig.set_splitting_ops_for_v1

            def set_splitting_ops_for_v1(self, *a, **k):
                orig(self, *a, **k)
                if getattr(self, "splitting_ops", None) is not None and \
                        "vllm::all_reduce" not in self.splitting_ops:
                    self.splitting_ops.append("vllm::all_reduce")

            CompilationConfig.set_splitting_ops_for_v1 = set_splitting_ops_for_v1
        except Exception as e:
            _debug("splitting-ops patch skipped: %s" % e)

    if _step(6):
        try:
            from . import quant

            _debug("registered quantization method %r" % quant.register())
        except Exception as e:
            _debug("quantization method not registered: %s" % e)


install()
