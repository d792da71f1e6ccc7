# SPDX-License-Identifier: MIT
"""Payload started by tools/blrun in test_blrun_cpu.py: checks the environment
the launcher promises (rank variables, no capabilities, no_new_privs), then
joins the "barlink" process group on CPU tensors and sums across ranks.
Counterpart of the reference's torch_ext/tests/payload_caps_check.py:7-31."""
import os
import sys

mode = sys.argv[1] if len(sys.argv) > 1 else "ok"
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
assert os.environ["MASTER_ADDR"] == "127.0.0.1" and int(os.environ["MASTER_PORT"]) > 0
assert os.environ.get("BL_SKIP_INIT") == "1" and os.environ.get("BL_PG_ID", "").startswith("blrun")
status = dict(line.split(":\t", 1) for line in open("/proc/self/status").read().splitlines() if ":\t" in line)
assert int(status["CapAmb"], 16) == 0, status["CapAmb"]
assert int(status["NoNewPrivs"]) == 1
if os.environ.get("BL_EXPECT_NO_CAPS") == "1":
    assert int(status["CapEff"], 16) == 0, status["CapEff"]
if mode == "fail" and rank == 1:
    sys.exit(5)

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

os.environ["BL_CPU_ONLY"] = "1"
from barlink_sm86_b200 import process_group as blpg  # noqa: E402

blpg.init_process_group(rank=rank, world_size=world)
t = torch.full((4,), float(rank + 1))
dist.all_reduce(t)
assert torch.all(t == sum(range(1, world + 1)))
if mode == "fail":
    import time
    time.sleep(60)  # the launcher must take this rank down when rank 1 fails
print("payload rank %d of %d ok, CapEff=%s" % (rank, world, status["CapEff"]), flush=True)
dist.destroy_process_group()
