#!/usr/bin/env bash
# Optimisation matrix: the same configuration under a set of flag combinations (communication back end, micro-batch,
# AttnRes off, Newton-Schulz presets, AdamW only, fp8, tensor parallelism); one record per run and a speed-up table.
#   tools/run_benchmark.sh                                   # configs/canary-3b.yaml, 60 steps per run
#   tools/run_benchmark.sh configs/proxy-benchmark.yaml      # another base configuration
#   tools/run_benchmark.sh configs/canary-3b.yaml --only native,nccl,fp8
set -euo pipefail
cd "$(dirname "$0")/.."
CFG="${1:-configs/canary-3b.yaml}"; [ $# -gt 0 ] && shift
exec python tools/benchmark_matrix.py matrix --config "${CFG}" --steps "${STEPS:-60}" "$@"
