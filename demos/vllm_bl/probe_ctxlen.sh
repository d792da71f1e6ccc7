#!/usr/bin/env bash
# SPDX-License-Identifier: MIT
# KV-capacity sweep: start vLLM at growing max_model_len and record how many
# tokens of KV cache it reports (fp8 KV, chunked prefill, one sequence).
# Usage: probe_ctxlen.sh [tp] ; BL_SHIM_OFF=1 for the NCCL baseline.
set -u
HERE="$(cd "$(dirname "$0")" && pwd)"
TP="${1:-2}"
for LEN in 32768 65536 98304 131072 196608 262144; do
  LOG="$HERE/probe_ctx_${LEN}.log"
  echo "##### probing max_model_len=$LEN $(date)"
  timeout 900 python "$HERE/bench_tp.py" --tp "$TP" --max-num-seqs 1 --gpu-mem 0.93 --num-prompts 1 \
    --prompt-tokens 512 --max-tokens 8 --max-model-len "$LEN" --kv-dtype fp8_e4m3 --chunked-prefill \
    --warm-repeat 0 --out-json "$HERE/probe_ctx_${LEN}.json" > "$LOG" 2>&1
  RC=$?
  KV=$(grep -oE "GPU KV cache size: [0-9,]+ tokens" "$LOG" | tail -1)
  echo "##### LEN=$LEN rc=$RC $KV"
  [ $RC -ne 0 ] && grep -iE "out of memory|no available memory|exceeds|error" "$LOG" | head -3
done
echo "##### sweep done $(date)"
