# SPDX-License-Identifier: MIT
"""With the repository root on PYTHONPATH, every interpreter start imports the
vLLM hook (same mechanism as the reference's root sitecustomize.py:9-13).  It
only acts when BL_SHIM=1 is set, so that unrelated python programs run from
this directory are left alone."""
import os

if os.environ.get("BL_SHIM") == "1":
    try:
        import vllm_barlink  # noqa: F401  (install() runs at import)
    except Exception as e:  # never break an unrelated interpreter start
        import sys

        sys.stderr.write("sitecustomize: vllm_barlink hook skipped: %s\n" % e)
