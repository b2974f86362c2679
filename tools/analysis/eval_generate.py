#!/usr/bin/env python
"""Evaluation generation pipeline (track 3): text samples for a prompt set from one or several
checkpoints, plus held-out perplexity on a flat uint16 token file.

    python tools/analysis/eval_generate.py --checkpoint ckpt.pt --name my-run
    python tools/analysis/eval_generate.py --checkpoints proxy-muon,proxy-attnres --n-samples 3
    python tools/analysis/eval_generate.py --checkpoint ckpt.pt --name t --no-ppl --temperature 0.8 --top-p 0.9

Writes ``<output-dir>/<run>/generations.json``.  Counterpart of the reference's
``scripts/analysis/eval_generate.py``.
"""
from __future__ import annotations

import argparse
import time

import torch
from _common import ROOT, add_checkpoint_args, load_yaml, open_model, run_dir, select_checkpoints, tokenizer, write_json

from kotodama_b200.eval import compute_perplexity, generate_text


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_checkpoint_args(ap)
    ap.add_argument("--prompt-set", default="standard")
    ap.add_argument("--prompts-file", default=str(ROOT / "configs" / "prompts.yaml"))
    ap.add_argument("--n-samples", type=int, default=1)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--no-ppl", action="store_true")
    ap.add_argument("--ppl-data", default="data/heldout.bin")
    ap.add_argument("--ppl-tokens", type=int, default=1_000_000)
    ap.add_argument("--seq-len", type=int, default=2048)
    a = ap.parse_args()
    prompts = load_yaml(a.prompts_file)[a.prompt_set]
    tok = tokenizer(a.tokenizer)
    for run, kw in select_checkpoints(a):
        model, meta = open_model(kw, a.device)
        torch.manual_seed(a.seed)
        t0 = time.time()
        gens = []
        for p in prompts:
            samples = [generate_text(model, tok, p, max_new_tokens=a.max_tokens, temperature=a.temperature,
                                     top_k=a.top_k, top_p=a.top_p, repetition_penalty=a.repetition_penalty)
                       for _ in range(a.n_samples)]
            gens.append({"prompt": p, "samples": samples})
        out = {"run": run, "checkpoint": str(kw["checkpoint"]), **{k: v for k, v in meta.items() if v is not None},
               "config": {"temperature": a.temperature, "top_k": a.top_k, "top_p": a.top_p, "max_tokens": a.max_tokens,
                          "repetition_penalty": a.repetition_penalty, "n_samples": a.n_samples, "prompt_set": a.prompt_set},
               "generations": gens, "generation_s": round(time.time() - t0, 2)}
        if not a.no_ppl:
            try:
                out["perplexity"] = compute_perplexity(model, a.ppl_data, seq_len=min(a.seq_len, model.config.max_position_embeddings),
                                                       max_tokens=a.ppl_tokens)
            except (FileNotFoundError, ValueError) as e:
                out["perplexity"] = {"error": str(e)}
        write_json(run_dir(a.output_dir, run) / "generations.json", out)
        print(f"{run}: {len(gens)} prompts x {a.n_samples} samples -> {run_dir(a.output_dir, run) / 'generations.json'}")


if __name__ == "__main__":
    main()
