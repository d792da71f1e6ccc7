# SPDX-License-Identifier: MIT
"""barlink for B200 -- Python front of the compiled extension.

Same role as the reference's package front
(torch_ext/barlink_sm86/__init__.py:15-119): the compiled module `_C` is
loaded lazily so that `import barlink_sm86_b200` works (and says what to do)
on a machine where the extension has not been built, the link op surface is
re-exported, and the chunked helpers `copy_large` / `allreduce_large` are
kept.  Differences: up to 8 ranks, `allreduce_` takes one pool tensor per
arena, and the new collectives (`allgather_into`, `reduce_scatter_into`,
`broadcast_`, `barrier`, `allreduce_rmsnorm`) are exported next to the old
ones.

Sub-packages: `ops` (kernel wrappers and their CPU oracles), `parallel`
(tensor-parallel linears), `models` (Qwen2-style decoder, MMDiT), `utils`.
"""
import importlib
import importlib.util
import os
import sys

__version__ = "0.1.0"

_HERE = os.path.dirname(os.path.abspath(__file__))
_C_MODULE = None
_C_ERROR = None


def _so_candidates():
    import torch

    tv = torch.__version__.split("+")[0].split(".")
    tagged = os.path.join(_HERE, "_build", "_C.torch%s%s.so" % (tv[0], tv[1]))
    return [tagged, os.path.join(_HERE, "_build", "_C.so")]


def load_extension(required=True):
    """Import the compiled module once; `required=False` returns None when it is missing."""
    global _C_MODULE, _C_ERROR
    if _C_MODULE is not None:
        return _C_MODULE
    if "barlink_sm86_b200._C" in sys.modules:  # adopted from an in-process build
        _C_MODULE = sys.modules["barlink_sm86_b200._C"]
        return _C_MODULE
    try:
        import torch  # noqa: F401  (also makes libc10/libtorch resolvable for the .so)
    except ImportError as e:  # pragma: no cover
        raise ImportError("barlink_sm86_b200 requires PyTorch: %s" % e) from e
    for path in _so_candidates():
        if os.path.exists(path):
            try:
                spec = importlib.util.spec_from_file_location("barlink_sm86_b200._C", path)
                mod = importlib.util.module_from_spec(spec)
                spec.loader.exec_module(mod)
                sys.modules["barlink_sm86_b200._C"] = mod
                _C_MODULE = mod
                return mod
            except ImportError as e:
                _C_ERROR = e
    if not required:
        return None
    raise ImportError(
        "barlink_sm86_b200: the compiled extension was not found (or failed to load: %s).\n"
        "Build it in-tree with:\n    python -m barlink_sm86_b200._build\n"
        "(needs nvcc with sm_100a support and the torch this interpreter imports)." % (_C_ERROR,)
    )


class _LazyC:
    """Attribute access loads the extension; importing this package never does."""

    def __getattr__(self, name):
        return getattr(load_extension(), name)


_C = _LazyC()


def _fwd(name):
    def call(*a, **kw):
        return getattr(load_extension(), name)(*a, **kw)

    call.__name__ = name
    call.__doc__ = "barlink_sm86_b200._C.%s" % name
    return call


init = _fwd("init")
init_peer = _fwd("init_peer")
shutdown = _fwd("shutdown")
info = _fwd("info")
empty = _fwd("empty")
free_ = _fwd("free_")
copy_ = _fwd("copy_")
allreduce_into = _fwd("allreduce_into")
allgather_into = _fwd("allgather_into")
reduce_scatter_into = _fwd("reduce_scatter_into")
broadcast_ = _fwd("broadcast_")
barrier = _fwd("barrier")
allreduce_rmsnorm = _fwd("allreduce_rmsnorm")
send_into = _fwd("send_into")
recv_into = _fwd("recv_into")
verify = _fwd("verify")
readback = _fwd("readback")
pool_move = _fwd("pool_move")
debug_flags = _fwd("debug_flags")
signal_probe = _fwd("signal_probe")
status = _fwd("status")
reset = _fwd("reset")
stats = _fwd("stats")
set_wait_timeout_ms = _fwd("set_wait_timeout_ms")


def allreduce_(*tensors):
    """Single-process all-reduce over pool tensors, one per arena.

    `allreduce_(a, b)` is the reference's two-GPU form; more arenas take more
    tensors (or one list)."""
    if len(tensors) == 1 and isinstance(tensors[0], (list, tuple)):
        tensors = tuple(tensors[0])
    return load_extension().allreduce_(list(tensors))


def _chunk_elems(itemsize, chunk_bytes):
    per = max(1, 16 // itemsize)
    return max(per, (max(16, chunk_bytes) // 16) * per)


def copy_large(dst, src, chunk_bytes=256 << 20):
    """Chunked `copy_` on the 16-byte granularity (reference: __init__.py:83-99)."""
    total = src.numel()
    if total == 0:
        return
    if src.element_size() != dst.element_size():
        raise TypeError("barlink copy_large: dtype mismatch")
    step = _chunk_elems(src.element_size(), chunk_bytes)
    for i in range(0, total, step):
        j = min(i + step, total)
        copy_(dst[i:j], src[i:j])


def allreduce_large(*tensors, chunk_bytes=None):
    """Chunked `allreduce_` for tensors above the per-call limit (reference: __init__.py:102-114)."""
    if len(tensors) == 1 and isinstance(tensors[0], (list, tuple)):
        tensors = tuple(tensors[0])
    total = tensors[0].numel()
    if total == 0:
        return
    if any(t.element_size() != tensors[0].element_size() for t in tensors):
        raise TypeError("barlink allreduce_large: dtype mismatch")
    if chunk_bytes is None:
        chunk_bytes = info()["max_chunk"]
    step = _chunk_elems(tensors[0].element_size(), chunk_bytes)
    for i in range(0, total, step):
        j = min(i + step, total)
        allreduce_([t[i:j] for t in tensors])


__all__ = [
    "init", "init_peer", "shutdown", "info", "empty", "free_", "copy_", "allreduce_",
    "allreduce_into", "allgather_into", "reduce_scatter_into", "broadcast_", "barrier",
    "allreduce_rmsnorm", "send_into", "recv_into", "copy_large", "allreduce_large", "verify",
    "readback", "pool_move", "debug_flags", "signal_probe", "status", "reset", "stats",
    "set_wait_timeout_ms", "load_extension",
]
