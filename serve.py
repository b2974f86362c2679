#!/usr/bin/env python
"""Inference server entry point.

    python serve.py --checkpoint checkpoints/run/step_00045775.pt [--device cuda] [--host 0.0.0.0] [--port 2222]
    torchrun --nproc-per-node 8 --master-addr 127.0.0.1 serve.py --model_size 3b ...    # tensor-parallel

Under ``torchrun`` the model is sharded over the ranks (tensor parallelism: heads, KV cache and MLP
columns); rank 0 hosts the HTTP app and drives the other ranks in lock-step.

Same flags as the reference server (``serve.py:601-615``: ``--checkpoint --device --compile --host
--port``; ``--compile`` is accepted and ignored, the native kernel path is always on) plus the
model description, which the reference hard-codes to its 108M proxy with the DD-v1 AttnRes
boundaries (``serve.py:50-72``) and which stays the default here.
"""
from __future__ import annotations

import argparse
import logging
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

from kotodama_b200.ckpt.manager import clean_state_dict, load_checkpoint_file  # noqa: E402
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.serve.app import create_app, load_tokenizer  # noqa: E402
from kotodama_b200.serve.engine import ServingEngine  # noqa: E402

logger = logging.getLogger("kotodama_b200.serve")

DEFAULT_CHECKPOINT = "checkpoints/lang-full-ddv1/step_00045775.pt"
TOKENIZER_NAME = "HuggingFaceTB/SmolLM2-135M"
DDV1_BOUNDARIES = "0,3,7,12,21,25"


def load_model(checkpoint: str, model_size: str, boundaries: str, n_blocks: int, attn_res: bool,
               random_init: bool = False) -> KotodamaModel:
    kw = dict(MODEL_PRESETS[model_size], z_loss_weight=0.0, attn_res=attn_res, attn_res_n_blocks=n_blocks)
    if attn_res and boundaries:
        kw["attn_res_boundaries"] = [int(x) for x in boundaries.split(",")]
    model = KotodamaModel(ModelConfig(**kw))
    if random_init:
        logger.warning("Serving random-init weights (--random_init)")
        return model
    from pathlib import Path
    path = Path(checkpoint)
    if not path.exists():
        raise FileNotFoundError(f"Checkpoint not found: {path}")
    ckpt = load_checkpoint_file(path, map_location="cpu")
    model.load_state_dict(clean_state_dict(ckpt.get("model", ckpt)), strict=True)
    logger.info("Checkpoint loaded (step %s, %s tokens)", ckpt.get("step", "?"), ckpt.get("tokens_consumed", "?"))
    return model


def main() -> None:
    ap = argparse.ArgumentParser(description="kotodama-b200 inference server")
    ap.add_argument("--checkpoint", default=DEFAULT_CHECKPOINT)
    ap.add_argument("--device", default="cuda", choices=["cuda", "cpu"])
    ap.add_argument("--compile", action="store_true", help="accepted for compatibility; no effect")
    ap.add_argument("--host", default="0.0.0.0")
    ap.add_argument("--port", type=int, default=2222)
    ap.add_argument("--model_size", default="proxy", choices=list(MODEL_PRESETS))
    ap.add_argument("--no_attn_res", action="store_true")
    ap.add_argument("--attn_res_boundaries", default=DDV1_BOUNDARIES)
    ap.add_argument("--attn_res_n_blocks", type=int, default=7)
    ap.add_argument("--max_batch", type=int, default=64)
    ap.add_argument("--prefill_batch_tokens", type=int, default=8192,
                    help="rows of one padded prefill pass shared by several prompts (0: one prompt per pass)")
    ap.add_argument("--max_ctx", type=int, default=None)
    ap.add_argument("--tokenizer", default=TOKENIZER_NAME)
    ap.add_argument("--random_init", action="store_true", help="serve random weights (smoke tests)")
    args = ap.parse_args()
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(levelname)s %(name)s: %(message)s")
    device = "cuda" if args.device == "cuda" and torch.cuda.is_available() else "cpu"
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    tp = None
    if world > 1:
        import torch.distributed as dist
        from kotodama_b200.serve.tp import ServeTP, TPLeader, run_follower
        local = int(os.environ.get("LOCAL_RANK", rank))
        if device == "cuda":
            torch.cuda.set_device(local)
            device = f"cuda:{local}"
            dist.init_process_group("nccl", device_id=torch.device(device))
        else:
            dist.init_process_group("gloo")
        tp = ServeTP()
    model = load_model(args.checkpoint, args.model_size, args.attn_res_boundaries, args.attn_res_n_blocks,
                       not args.no_attn_res, args.random_init)
    engine = ServingEngine(model, device=device, dtype=torch.bfloat16 if device.startswith("cuda") else torch.float32,
                           max_batch=args.max_batch, max_ctx=args.max_ctx, tp=tp,
                           prefill_batch_tokens=args.prefill_batch_tokens)
    if tp is not None and rank > 0:
        run_follower(engine, tp)
        return
    if tp is not None:
        engine = TPLeader(engine, tp)
    tok = load_tokenizer(args.tokenizer)
    logger.info("Device %s, tokenizer %s, paged KV cache with %d pages", device, type(tok).__name__,
                engine.cache.num_pages)
    import uvicorn
    uvicorn.run(create_app(engine, tok, model_name=f"kotodama-{args.model_size}", checkpoint=args.checkpoint or ""), host=args.host, port=args.port)


if __name__ == "__main__":
    main()
