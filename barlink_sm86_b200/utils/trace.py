# SPDX-License-Identifier: MIT
"""Op-level tracer: a ring buffer of (op, shapes, bytes, device time) for every
call that goes through `barlink_sm86_b200.ops` and `TPComm`, with optional
NVTX ranges for timeline tools.

    with OpTrace() as t:
        engine.step()
    print(t.table())          # per-op count / total / mean microseconds
    t.dump("trace.json")

`BL_TRACE=1` in the environment turns tracing on for the whole process (the
buffer is then at `barlink_sm86_b200.utils.trace.ACTIVE`); `BL_TRACE_SIZE`
sets the ring capacity (default 65536 records); `BL_NVTX=1` adds NVTX ranges.
Timing uses one CUDA event pair per call on the current stream and is read
lazily, so tracing does not synchronise the device; it cannot run inside a
CUDA-graph capture (events would be captured) and says so.
"""
import collections
import json
import os
import time

import torch

ACTIVE = None
_COMM_METHODS = ("all_reduce", "all_gather_cols", "all_gather_rows", "allreduce_rmsnorm", "argmax_vocab_parallel")


def _describe(args):
    shapes, nbytes = [], 0
    for a in args:
        if isinstance(a, torch.Tensor):
            shapes.append(list(a.shape))
            nbytes += a.numel() * a.element_size()
        elif hasattr(a, "shape") and hasattr(a, "numel"):
            shapes.append(list(a.shape))
    return shapes, nbytes


class OpTrace:
    def __init__(self, capacity=None, nvtx=None):
        self.capacity = capacity or int(os.environ.get("BL_TRACE_SIZE", "65536"))
        self.nvtx = (os.environ.get("BL_NVTX", "0") == "1") if nvtx is None else nvtx
        self.records = collections.deque(maxlen=self.capacity)
        self._saved = []

    # ---- patching --------------------------------------------------------
    def _wrap(self, name, fn):
        trace = self

        def wrapped(*args, **kwargs):
            cuda = any(isinstance(a, torch.Tensor) and a.is_cuda for a in args)
            if cuda and torch.cuda.is_current_stream_capturing():
                raise RuntimeError("barlink: OpTrace cannot record inside a CUDA-graph capture")
            shapes, nbytes = _describe(args)
            if trace.nvtx and cuda:
                torch.cuda.nvtx.range_push("bl." + name)
            if cuda:
                s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                s.record()
                out = fn(*args, **kwargs)
                e.record()
                trace.records.append({"op": name, "shapes": shapes, "bytes": nbytes, "events": (s, e)})
            else:
                t0 = time.perf_counter()
                out = fn(*args, **kwargs)
                trace.records.append({"op": name, "shapes": shapes, "bytes": nbytes,
                                      "us": (time.perf_counter() - t0) * 1e6})
            if trace.nvtx and cuda:
                torch.cuda.nvtx.range_pop()
            return out

        wrapped.__wrapped__ = fn
        return wrapped

    def start(self):
        from .. import ops
        from ..parallel import comm as comm_mod
        for name in ops.__all__:
            fn = getattr(ops, name, None)
            if callable(fn) and not isinstance(fn, type) and name not in ("tile_weight", "untile_weight", "k_splits"):
                self._saved.append((ops, name, fn))
                setattr(ops, name, self._wrap(name, fn))
        for name in _COMM_METHODS:
            fn = getattr(comm_mod.TPComm, name)
            self._saved.append((comm_mod.TPComm, name, fn))
            setattr(comm_mod.TPComm, name, self._wrap("comm." + name, fn))
        return self

    def stop(self):
        for owner, name, fn in reversed(self._saved):
            setattr(owner, name, fn)
        self._saved = []
        self.resolve()

    def __enter__(self):
        return self.start()

    def __exit__(self, *exc):
        self.stop()
        return False

    # ---- reading ---------------------------------------------------------
    def resolve(self):
        """Turn event pairs into microseconds (synchronises once)."""
        if any("events" in r for r in self.records) and torch.cuda.is_available():
            torch.cuda.synchronize()
        for r in self.records:
            ev = r.pop("events", None)
            if ev is not None:
                r["us"] = ev[0].elapsed_time(ev[1]) * 1e3

    def summary(self):
        self.resolve()
        agg = collections.OrderedDict()
        for r in self.records:
            a = agg.setdefault(r["op"], {"count": 0, "us": 0.0, "bytes": 0})
            a["count"] += 1
            a["us"] += r["us"]
            a["bytes"] += r["bytes"]
        return agg

    def table(self):
        agg = self.summary()
        total = sum(a["us"] for a in agg.values()) or 1.0
        lines = ["%-28s %8s %12s %10s %6s" % ("op", "calls", "total us", "mean us", "%")]
        for op, a in sorted(agg.items(), key=lambda kv: -kv[1]["us"]):
            lines.append("%-28s %8d %12.1f %10.2f %6.1f" % (op, a["count"], a["us"], a["us"] / a["count"],
                                                         100.0 * a["us"] / total))
        return "\n".join(lines)

    def dump(self, path):
        self.resolve()
        with open(path, "w") as f:
            json.dump({"records": list(self.records), "summary": self.summary()}, f)


def link_stats():
    """The link core's counter block (ops, bytes, algorithm chosen, timeouts),
    or {} when the extension or the link is not up."""
    try:
        from .. import load_extension
        return dict(load_extension().stats())
    except Exception:
        return {}


if os.environ.get("BL_TRACE", "0") == "1" and ACTIVE is None:
    ACTIVE = OpTrace().start()
