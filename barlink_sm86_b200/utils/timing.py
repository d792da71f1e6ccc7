# SPDX-License-Identifier: MIT
"""Device timing with CUDA events on the launching stream."""
import torch

_flush_buf = {}


def flush_l2(device=None, nbytes=256 << 20):
    """Overwrite a buffer larger than the 126 MB L2 so the next kernel starts cold."""
    dev = torch.device(device if device is not None else torch.cuda.current_device())
    key = (dev, nbytes)
    if key not in _flush_buf:
        _flush_buf[key] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
    _flush_buf[key].zero_()


def cuda_time_us(fn, warmup=3, iters=10, flush=True, reduce="median"):
    """Time fn() on the current stream: `warmup` untimed calls, then `iters`
    calls each bracketed by events (L2 flushed before each when `flush`).
    Returns microseconds (median, mean or min)."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        if flush:
            flush_l2()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        fn()
        e.record()
        torch.cuda.synchronize()
        ts.append(s.elapsed_time(e) * 1e3)
    ts.sort()
    if reduce == "min":
        return ts[0]
    if reduce == "mean":
        return sum(ts) / len(ts)
    return ts[len(ts) // 2]


def max_over_ranks(value, group=None, device=None):
    """A multi-GPU step is as slow as its slowest rank."""
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return float(value)
    dev = device if device is not None else ("cuda" if torch.cuda.is_available() and dist.get_backend(group) != "gloo"
                                             else "cpu")
    t = torch.tensor([float(value)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX, group=group)
    return float(t.item())
