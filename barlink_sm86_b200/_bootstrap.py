# SPDX-License-Identifier: MIT
"""Bootstrap behind `tools/blrun`.

Same contract as the reference's bootstrap (torch_ext/barlink_sm86/
_bootstrap.py:14-29): with BL_SKIP_INIT=1 the script runs as is (SPMD ranks
bring the link up themselves through `init_process_group`); otherwise the
link is initialised in single-process mode for BL_DEVICES (default "0,1" when
two GPUs are present, else "0") with BL_POOL_MB (default 64) MiB per arena,
and then the script runs."""
import os
import runpy
import sys


def main():
    if len(sys.argv) < 2:
        sys.stderr.write("usage: python -m barlink_sm86_b200._bootstrap script.py [args...]\n")
        sys.exit(2)
    if os.environ.get("BL_SKIP_INIT") != "1":
        import torch

        import barlink_sm86_b200 as bl

        default = "0,1" if torch.cuda.is_available() and torch.cuda.device_count() >= 2 else "0"
        devs = [int(x) for x in os.environ.get("BL_DEVICES", default).split(",") if x != ""]
        pool_mb = int(os.environ.get("BL_POOL_MB", "64"))
        bl.init(devices=devs, pool_mb=pool_mb)
    script = sys.argv[1]
    sys.argv = sys.argv[1:]
    runpy.run_path(script, run_name="__main__")


if __name__ == "__main__":
    main()
