# SPDX-License-Identifier: MIT
"""torch.distributed backend "barlink".

Capability parity with the reference's backend module
(torch_ext/barlink_sm86/process_group.py:571-615: `_resolve_device`,
`_creator`, `register`, `init_process_group`), with these differences:

* the Backend class itself is C++ (`_C.BarlinkBackend`); this module only
  resolves the device, brings the link up and hands both to the class;
* 2..8 ranks instead of exactly 2; groups of one member are local no-ops;
  groups of 2..world-1 members are served by the gloo companion (CUDA tensors
  are staged through host memory: functional, not fast);
* the rendezvous socket path is agreed through the c10d store instead of a
  fixed /tmp name, so two jobs on one host cannot collide
  (`BL_SOCK_PATH` still overrides it);
* CPU tensors are served by a gloo companion, which lets the same group carry
  host-side plumbing (and lets the whole stack be tested without a GPU).

Environment: BL_POOL_MB (default 1024), BL_DEVICE / LOCAL_RANK, BL_SOCK_PATH,
BL_PG_ID, BL_CPU_ONLY=1 (never touch CUDA), BL_PG_DEBUG=1, BL_NVLS=1.
"""
import os
import sys
import tempfile

import torch
import torch.distributed as dist

from . import load_extension

BACKEND_NAME = "barlink"
_registered = False
_world_link_size = None  # size of the group that owns the link


def _debug(msg):
    if os.environ.get("BL_PG_DEBUG") == "1":
        sys.stderr.write("[barlink pg %s] %s\n" % (os.environ.get("RANK", "?"), msg))


def _resolve_device():
    """CUDA device of this rank: BL_DEVICE, else LOCAL_RANK, else the current device."""
    for var in ("BL_DEVICE", "LOCAL_RANK"):
        v = os.environ.get(var)
        if v is not None and v != "":
            return torch.device("cuda", int(v) % max(1, torch.cuda.device_count()))
    return torch.device("cuda", torch.cuda.current_device())


def _cuda_usable():
    if os.environ.get("BL_CPU_ONLY") == "1":
        return False
    try:
        return torch.cuda.is_available() and torch.cuda.device_count() > 0
    except Exception:
        return False


def _agree_socket_path(store, rank):
    forced = os.environ.get("BL_SOCK_PATH")
    if forced:
        return forced
    key = "barlink/sock"
    if rank == 0:
        tag = os.environ.get("BL_PG_ID") or "%d" % os.getpid()
        # a directory only this user can enter, so that nobody else can put a socket of that name there
        # (rank 0 also checks the uid of every process that connects)
        d = tempfile.mkdtemp(prefix="barlink-pg-%d-" % os.getuid())
        os.chmod(d, 0o700)
        import atexit
        import shutil
        atexit.register(shutil.rmtree, d, True)
        path = os.path.join(d, "%s.sock" % tag)
        store.set(key, path)
        return path
    return store.get(key).decode()


def _creator(dist_backend_opts, backend_opts):
    global _world_link_size
    C = load_extension()
    store = dist_backend_opts.store
    rank = dist_backend_opts.group_rank
    size = dist_backend_opts.group_size
    timeout = dist_backend_opts.timeout
    if size == 1:
        # a group of one never touches the link (reference: process_group.py:523-565)
        return C.BarlinkBackend(rank, size, None, False)

    cpu = dist.ProcessGroupGloo(dist.PrefixStore("barlink/gloo", store), rank, size, timeout=timeout)
    use_link = False
    if _cuda_usable():
        info = C.info()
        world = dist.get_world_size() if dist.is_initialized() else size
        if info.get("initialized") and info.get("peer_mode"):
            use_link = info["world"] == size
        elif size == world or not dist.is_initialized():
            device = _resolve_device()
            torch.cuda.set_device(device)
            pool_mb = int(os.environ.get("BL_POOL_MB", "1024"))
            sock = _agree_socket_path(store, rank)
            _debug("init_peer device=%s pool_mb=%d sock=%s rank=%d/%d" % (device, pool_mb, sock, rank, size))
            C.init_peer(device.index, pool_mb, sock, rank, size)
            _world_link_size = size
            use_link = True
        if not use_link:
            _debug("group of %d ranks inside a link of %s: CPU service only" % (size, info.get("world")))
    return C.BarlinkBackend(rank, size, cpu, use_link)


def register():
    """Register the backend name once (idempotent)."""
    global _registered
    if _registered:
        return
    dist.Backend.register_backend(BACKEND_NAME, _creator, extended_api=True, devices=["cpu", "cuda"])
    _registered = True


def init_process_group(*args, **kwargs):
    """`torch.distributed.init_process_group` with backend "barlink"."""
    register()
    kwargs.setdefault("backend", BACKEND_NAME)
    return dist.init_process_group(*args, **kwargs)


def backend_of(group=None):
    """The `_C.BarlinkBackend` object behind a process group (for its path counters)."""
    group = group or dist.group.WORLD
    for dev in ("cuda", "cpu"):
        try:
            return group._get_backend(torch.device(dev))
        except Exception:
            continue
    return None
