#!/bin/sh
# SPDX-License-Identifier: MIT
# Make every interpreter of a virtualenv import the barlink hook at start:
#   vllm_barlink/install_pth.sh <venv-dir>
# writes <site-packages>/vllm_barlink.pth (remove that file to undo).
set -eu
VENV="${1:?usage: install_pth.sh <venv-dir>}"
ROOT="$(cd "$(dirname "$0")/.." && pwd)"
"$VENV/bin/python" - "$ROOT" <<'PYEOF'
import site, sys
root = sys.argv[1]
sp = site.getsitepackages()[0]
with open(sp + "/vllm_barlink.pth", "w") as f:
    f.write("import sys; sys.path.insert(0, %r); import vllm_barlink\n" % root)
print("installed %s/vllm_barlink.pth" % sp)
PYEOF
