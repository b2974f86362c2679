#!/usr/bin/env bash
# Throughput canaries (3B and 8B by default) on this node: logs, per-model summaries, wall-clock estimates.
#   tools/run_canary.sh                 # both models on all GPUs
#   tools/run_canary.sh 3b              # one model
#   tools/run_canary.sh 8b 1            # one model on one GPU
#   tools/run_canary.sh 3b 8 -- --fp8   # flags after -- go to every run
set -euo pipefail
cd "$(dirname "$0")/.."
MODEL="${1:-both}"; [ $# -gt 0 ] && shift
GPUS="${1:-0}"; [ $# -gt 0 ] && shift
case "${MODEL}" in
  both) MODELS="3b,8b" ;;
  3b|8b) MODELS="${MODEL}" ;;
  *) echo "usage: $0 [3b|8b|both] [gpus] [-- extra train flags]"; exit 1 ;;
esac
exec python tools/benchmark_matrix.py canary --models "${MODELS}" --gpus "${GPUS}" "$@"
