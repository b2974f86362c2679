#!/usr/bin/env bash
# Perplexity of a checkpoint on a token file:  tools/run_eval.sh <checkpoint> <tokens.bin> [section]
set -euo pipefail
cd "$(dirname "$0")/.."
python - "$@" <<'PY'
import json, sys, torch
from kotodama_b200.eval import compute_perplexity, load_model
ckpt, data = sys.argv[1], sys.argv[2]
section = sys.argv[3] if len(sys.argv) > 3 else "proxy"
dev = "cuda" if torch.cuda.is_available() else "cpu"
model, meta = load_model(ckpt, section=section, device=dev, dtype=torch.bfloat16 if dev == "cuda" else None)
print(json.dumps({"checkpoint": ckpt, **meta, **compute_perplexity(model, data, seq_len=2048)}))
PY
