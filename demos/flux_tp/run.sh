#!/usr/bin/env bash
# SPDX-License-Identifier: MIT
# MMDiT tensor-parallel demo: TP=1, then TP=N over the link and over NCCL with
# the same kernels, then the comparisons.  Usage: run.sh [N] [out-dir] [extra worker flags]
set -euo pipefail
HERE="$(cd "$(dirname "$0")" && pwd)"
N="${1:-2}"
OUT="${2:-$HERE/results}"
shift $(( $# > 2 ? 2 : $# ))
PORT="${PORT:-29531}"
LIMIT="${LIMIT:-600}"   # seconds per run; a stuck run ends instead of holding the GPUs

run_tp() {  # backend tag
  timeout "$LIMIT" python -m torch.distributed.run --nnodes=1 --nproc-per-node "$N" \
    --master-addr 127.0.0.1 --master-port "$PORT" "$HERE/worker.py" \
    --backend "$1" --tag "$2" --out "$OUT" "${@:3}"
}

timeout "$LIMIT" python "$HERE/worker.py" --out "$OUT" --tag tp1 "$@"
if [ "$N" -gt 1 ]; then
  run_tp barlink "tp${N}" "$@"
  # the NCCL arm is a baseline: its failure must not hide the link's results
  NCCL_NVLS_ENABLE="${NCCL_NVLS_ENABLE:-0}" run_tp nccl "tp${N}nccl" "$@" > "$OUT/tp${N}nccl.log" 2>&1 \
    || echo "NCCL arm exited non-zero (see $OUT/tp${N}nccl.log)"
  grep -E "^\[tp" "$OUT/tp${N}nccl.log" || true
  python "$HERE/compare.py" --dir "$OUT" --left-tag tp1 --right-tag "tp${N}"
  if [ -f "$OUT/stats_tp${N}nccl.json" ]; then
    python "$HERE/compare.py" --dir "$OUT" --left-tag "tp${N}nccl" --right-tag "tp${N}"
  fi
fi
