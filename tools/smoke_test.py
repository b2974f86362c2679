#!/usr/bin/env python
"""Single-device sanity run of the whole training stack, a minute on a CPU:

1. tiny AttnRes model + Muon/AdamW through the executor, 50 steps on a fixed batch: the loss must
   fall (fresh uniform-random tokens cannot be learned, so the reference's variant of this check,
   ``scripts/utils/smoke_test.py:18-128``, only sees noise around ln(vocab));
2. the parameter split of the hybrid optimizer (2-D projections -> Muon, the rest -> AdamW);
3. ``reinit_mlps`` (the NCA -> language transition): the evaluation loss must rise;
4. ``reinit_embeddings(2048)``: new vocabulary size in the embedding and the config;
5. a checkpoint round trip: save, reload into a fresh model, same evaluation loss.

    python tools/smoke_test.py [--device cpu|cuda] [--steps 50]
"""
import argparse
import os
import sys
import tempfile
import time

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.ckpt.manager import CheckpointManager  # noqa: E402
from kotodama_b200.config import ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.optim.muon import HybridScheduler, split_params  # noqa: E402


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--steps", type=int, default=50)
    a = ap.parse_args()
    dev = a.device
    dtype = torch.bfloat16 if dev.startswith("cuda") else torch.float32
    cfg = ModelConfig(hidden_size=256, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=64,
                      intermediate_size=512, vocab_size=1024, max_position_embeddings=2048, attn_res=True,
                      attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    muon_p, adamw_p = split_params(model)
    n_m, n_a = sum(p.numel() for p in muon_p), sum(p.numel() for p in adamw_p)
    print(f"parameters: Muon {n_m:,} in {len(muon_p)} matrices ({100 * n_m / (n_m + n_a):.1f} %), "
          f"AdamW {n_a:,} in {len(adamw_p)} tensors")
    ok = len(muon_p) == 7 * cfg.num_layers and all(p.ndim == 2 for p in muon_p)
    eng = TrainEngine(model, device=dev, dtype=dtype)
    ids = torch.randint(0, cfg.vocab_size, (4, 256))
    t0 = time.time()
    losses = [float(eng.train_step([ids])["loss"]) for _ in range(a.steps)]
    dt = time.time() - t0
    print(f"[1] {a.steps} steps on a fixed batch: loss {losses[0]:.3f} -> {losses[-1]:.3f} "
          f"({a.steps / dt:.1f} steps/s, {a.steps * ids.numel() / dt:,.0f} tok/s on {dev})")
    ok = ok and losses[-1] < losses[0] - 0.5
    eng.check()
    with torch.no_grad():
        before = float(eng.eval_loss(ids))
        with tempfile.TemporaryDirectory() as d:
            sched = HybridScheduler(eng.muon_opt, eng.adamw_opt, warmup_steps=2, total_steps=a.steps)
            CheckpointManager(d, rank=0).save(a.steps - 1, model, eng.muon_opt, eng.adamw_opt, sched, a.steps * ids.numel())
            fresh = KotodamaModel(cfg)
            e2 = TrainEngine(fresh, device=dev, dtype=dtype)
            st = CheckpointManager(d, rank=0).load_latest(fresh, e2.muon_opt, e2.adamw_opt, torch.device(dev))
            e2.after_load()
            again = float(e2.eval_loss(ids))
        print(f"[5] checkpoint round trip: eval loss {before:.4f} -> {again:.4f} (step {st['step']})")
        ok = ok and abs(before - again) < 1e-2
        model.reinit_mlps()
        eng.after_load()
        after = float(eng.eval_loss(ids))
    print(f"[3] reinit_mlps: eval loss {before:.3f} -> {after:.3f}")
    ok = ok and after > before
    fresh = KotodamaModel(cfg)
    fresh.reinit_embeddings(2048)
    print(f"[4] reinit_embeddings(2048): embedding {tuple(fresh.embed_tokens.weight.shape)}, config vocab {fresh.config.vocab_size}")
    ok = ok and fresh.embed_tokens.weight.shape[0] == 2048 and fresh.config.vocab_size == 2048
    print("SMOKE TEST", "PASSED" if ok else "FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
