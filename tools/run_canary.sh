#!/usr/bin/env bash
# Run a canary config and summarise throughput from the step lines (p5 / median / p95 tok/s, peak memory, last loss).
#   tools/run_canary.sh configs/canary-3b.yaml [extra train flags]
set -euo pipefail
cd "$(dirname "$0")/.."
CFG="$1"; shift || true
NAME="$(basename "${CFG}" .yaml)"
LOG="logs/${NAME}-$(date +%Y%m%d-%H%M%S).log"
mkdir -p logs
tools/run_train.sh --config "${CFG}" "$@" 2>&1 | tee "${LOG}"
python tools/extract_benchmark_results.py "${LOG}"
