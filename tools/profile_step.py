#!/usr/bin/env python
"""Device time of the phases of one training step (forward+backward, gradient clip/norm, Muon,
AdamW), by wrapping the executor's ops and communication hooks with CUDA events.

    python tools/profile_step.py --model proxy --micro_batch 4 --seq 2048
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.monitor.profiler import PhaseTimer  # noqa: E402
from kotodama_b200.utils.optimer import TimedOps  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="proxy")
    ap.add_argument("--micro_batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--steps", type=int, default=3)
    a = ap.parse_args()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=True, attn_res_n_blocks=7 if a.model not in ("tiny", "smoke") else 2)
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    eng = TrainEngine.from_meta(model, cfg, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq))
    for _ in range(2):
        eng.train_step([ids])
    timer = PhaseTimer(dev == "cuda")
    for _ in range(a.steps):
        with timer.phase("FULL_STEP"):
            with timer.phase("FORWARD_BACKWARD"):
                eng.forward_backward(ids.to(eng.device))
            with timer.phase("OPTIMIZER_STEP"):
                eng.optimizer_step()
    for k, v in timer.totals_ms().items():
        print(f"{k:<20}{v / a.steps:>10.2f} ms/step")
    if dev == "cuda":
        plain = eng.ops
        eng.ops = TimedOps(plain)
        eng.train_step([ids])
        print(eng.ops.table(1))


if __name__ == "__main__":
    main()
