#!/usr/bin/env python
"""Single-device sanity run: tiny model + hybrid optimizer for 50 steps (loss must fall on a
fixed batch), then ``reinit_mlps`` (loss rises) and ``reinit_embeddings(2048)``."""
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.config import ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402


def main() -> int:
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    cfg = ModelConfig(hidden_size=256, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=64,
                      intermediate_size=512, vocab_size=1024, max_position_embeddings=2048, attn_res=True,
                      attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    eng = TrainEngine(model, device=dev, dtype=torch.bfloat16 if dev == "cuda" else torch.float32)
    ids = torch.randint(0, cfg.vocab_size, (4, 256))
    losses = [float(eng.train_step([ids])["loss"]) for _ in range(50)]
    print(f"loss {losses[0]:.3f} -> {losses[-1]:.3f}")
    ok = losses[-1] < losses[0]
    with torch.no_grad():
        before = float(eng.eval_loss(ids))
        model.reinit_mlps()
        after = float(eng.eval_loss(ids))
    print(f"reinit_mlps: eval loss {before:.3f} -> {after:.3f}")
    ok = ok and after > before
    fresh = KotodamaModel(cfg)
    fresh.reinit_embeddings(2048)
    ok = ok and fresh.embed_tokens.weight.shape[0] == 2048 and fresh.config.vocab_size == 2048
    print("SMOKE TEST", "PASSED" if ok else "FAILED")
    return 0 if ok else 1


if __name__ == "__main__":
    sys.exit(main())
