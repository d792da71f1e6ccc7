# SPDX-License-Identifier: MIT
"""Trampoline: run a vLLM script with the barlink hook installed.

    python vllm_barlink/entry.py demos/vllm_bl/bench_serving.py [args...]

The reference's trampoline re-executes the script under a second virtualenv so
that ambient capabilities reach vLLM's workers (vllm_barlink/entry.py:13-22
there).  Nothing here needs a capability; what has to reach the workers is the
hook itself.  vLLM starts its workers as fresh interpreters, so the hook is
put on PYTHONPATH as a `sitecustomize` (the repository root holds one), BL_SHIM=1
switches that sitecustomize on for the script and every interpreter it spawns, and
the script is re-executed under $BL_VLLM_PYTHON (default: this interpreter).
BL_SHIM_OFF=1 leaves the hook out (the NCCL arm of an A/B run)."""
import os
import sys


def main():
    if len(sys.argv) < 2:
        sys.stderr.write("usage: entry.py <script.py> [args...]\n")
        sys.exit(2)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    old = os.environ.get("PYTHONPATH", "")
    if root not in old.split(os.pathsep):
        os.environ["PYTHONPATH"] = root + (os.pathsep + old if old else "")
    if os.environ.get("BL_SHIM_OFF") != "1":
        os.environ["BL_SHIM"] = "1"
    py = os.environ.get("BL_VLLM_PYTHON", sys.executable)
    os.execv(py, [py] + sys.argv[1:])


if __name__ == "__main__":
    main()
