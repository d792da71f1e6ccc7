#!/bin/sh
# SPDX-License-Identifier: MIT
# Latency suite on N GPUs (default 2): raw link, process group on barlink and on
# NCCL, p2p.  Usage: bench/latency/run_all.sh [N]
set -u
N="${1:-2}"
HERE="$(cd "$(dirname "$0")" && pwd)"
LIMIT="${LIMIT:-180}"   # seconds per program: a stuck run ends instead of holding the GPUs
RUN="timeout $LIMIT python -m torch.distributed.run --nnodes=1 --nproc-per-node $N --master-addr 127.0.0.1"
$RUN --master-port 29601 "$HERE/link_lat.py"
for B in barlink nccl; do
  $RUN --master-port 29602 "$HERE/pg_lat.py" --backend $B
  $RUN --master-port 29603 "$HERE/pg_bw.py" --backend $B
  $RUN --master-port 29604 "$HERE/pg_p2p_lat.py" --backend $B
done
