#!/usr/bin/env bash
# Optimisation matrix: the same canary under a set of flag combinations; one summary line each.
set -euo pipefail
cd "$(dirname "$0")/.."
CFG="${1:-configs/canary-3b.yaml}"
declare -A RUNS=(
  [native]=""
  [nccl]="--backend nccl"
  [mb8]="--micro_batch_size 8"
  [no_attnres]="--no_attn_res"
  [original_ns]="--muon_ns_coefficients original"
  [adamw_only]="--adamw_only"
  [fp8]="--fp8"
  [tp8]="--tp_size 8 --sequence_parallel"
)
mkdir -p logs
for name in "${!RUNS[@]}"; do
  LOG="logs/bench-${name}.log"
  echo "== ${name}: ${RUNS[$name]}"
  tools/run_train.sh --config "${CFG}" --total_steps 60 --checkpoint_dir "checkpoints/bench-${name}" ${RUNS[$name]} > "${LOG}" 2>&1 || echo "   failed (see ${LOG})"
  python tools/extract_benchmark_results.py "${LOG}" || true
done
