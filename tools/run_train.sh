#!/usr/bin/env bash
# Launch training on all GPUs of this node:  tools/run_train.sh --config configs/canary-3b.yaml [--flag ...]
set -euo pipefail
cd "$(dirname "$0")/.."
NGPU="${NGPU:-$(nvidia-smi -L 2>/dev/null | wc -l)}"
[ "${NGPU}" -ge 1 ] || NGPU=1
export OMP_NUM_THREADS="${OMP_NUM_THREADS:-8}"
exec python -m torch.distributed.run --nnodes=1 --nproc-per-node "${NGPU}" --master-addr 127.0.0.1 \
    --master-port "${MASTER_PORT:-29500}" train.py "$@"
