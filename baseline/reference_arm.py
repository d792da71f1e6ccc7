# SPDX-License-Identifier: MIT
"""`bench.py --impl reference`: the unmodified reference, installed under
baseline/_ref, through its own public API.

What the install gives on a B200 box: `barlink_sm86._C` builds for sm_100
from the reference's torch_ext (installed from a copy, because its setup.py
builds in place), so its W8A16 kernels are callable.  Its transport cannot
come up: `bl.init` / `bl.init_peer` need the patched NVIDIA kernel module and
the dmabuf_holder device (/dev/dmabuf_holder), neither of which exists on an
NVSwitch box.  Its decode harness (demos/qwen_tp/qwen38_int8/worker.py) loads
a Qwen3.8-27B INT8 checkpoint from disk through HF transformers; there is no
network and no checkpoint here, and the harness has no random-init path.  The
headline metric (Qwen2.5-7B-shape TP decode tokens/s) therefore cannot be
produced by the reference's stock code path; this arm says so in one line.
`baseline/nccl_decode.py` restates the reference's NCCL branch (F.linear +
dist.all_reduce hooks + vocab-parallel head, CUDA-graphed) for the same model
shape and is the number to compare against instead.
"""
import json
import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def probe():
    """(importable, transport_possible, detail)"""
    if not os.path.isdir(os.path.join(REF, "barlink_sm86")):
        return False, False, "baseline/_ref/barlink_sm86 is not installed"
    transport = os.path.exists("/dev/dmabuf_holder")
    return True, transport, "installed"


def run_reference(args):
    importable, transport, detail = probe()
    if not importable:
        why = "reference not installed: %s" % detail
    elif not transport:
        why = ("reference transport needs the patched NVIDIA driver and /dev/dmabuf_holder (absent on this box), "
               "and its decode harness needs the Qwen3.8-27B INT8 checkpoint (no network); only its W8A16 "
               "kernels run here (see bench/w8a16_bench.py); NCCL+cuBLAS restatement: baseline/nccl_decode.py")
    else:
        why = "reference decode harness needs the Qwen3.8-27B INT8 checkpoint, which is not on this box"
    print(json.dumps({"impl": "reference", "unavailable": why}))
    return 0


if __name__ == "__main__":
    sys.exit(run_reference(None))
