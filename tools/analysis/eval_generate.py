#!/usr/bin/env python
"""Evaluation generation pipeline (track 3): text samples for a prompt set from one or several
checkpoints, plus held-out perplexity on a flat uint16 token file.

    python tools/analysis/eval_generate.py --checkpoint ckpt.pt --name my-run
    python tools/analysis/eval_generate.py --checkpoints proxy-muon,proxy-attnres --n-samples 3 --combined
    python tools/analysis/eval_generate.py --checkpoint ckpt.pt --name t --no-ppl --temperature 0.8 --top-p 0.9
    python tools/analysis/eval_generate.py --checkpoint ckpt.pt --name t --temperatures 0.3,0.7,1.0   # temperature matrix

Writes ``<output-dir>/<run>/generations.json`` per run: the samples grouped by prompt (what the text-quality
track reads), one record per sample (tokens, what ended it, seconds), the generation settings and the
perplexity.  ``--temperatures`` repeats the whole set at several temperatures (``generations_t<T>.json`` each and a
``temperature_matrix.json`` with perplexity-independent sample statistics per temperature); ``--combined`` also
writes one file with all runs side by side (``<output-dir>/<a>_vs_<b>/generations.json``).  A checkpoint that is
missing or does not load is skipped with a message, the others still run.  Counterpart of the reference's
``scripts/analysis/eval_generate.py``.
"""
from __future__ import annotations

import argparse
import time
from pathlib import Path

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
    ap.add_argument("--ppl-data", "--eval-data", dest="ppl_data", default="data/heldout.bin")
    ap.add_argument("--max-seqs", type=int, default=None, help="perplexity over this many sequences (sets --ppl-tokens to max-seqs x seq-len)")
    ap.add_argument("-o", "--output", default=None, help="also write the last run's generations file to this path")
    ap.add_argument("--ppl-tokens", type=int, default=1_000_000)
    ap.add_argument("--seq-len", type=int, default=2048)
    ap.add_argument("--temperatures", default=None, help="comma-separated: run the whole set at each of these temperatures")
    ap.add_argument("--combined", action="store_true", help="also write one file with all runs side by side")
    a = ap.parse_args()
    if a.max_seqs:
        a.ppl_tokens = a.max_seqs * a.seq_len
    prompts = load_yaml(a.prompts_file)[a.prompt_set]
    tok = tokenizer(a.tokenizer)
    temps = [float(t) for t in a.temperatures.split(",")] if a.temperatures else [a.temperature]
    done: list[dict] = []
    for run, kw in select_checkpoints(a):
        if not Path(str(kw["checkpoint"])).exists():
            print(f"{run}: {kw['checkpoint']} not found, skipped")
            continue
        try:
            model, meta = open_model(kw, a.device)
        except Exception as e:                               # a damaged file must not stop the other runs
            print(f"{run}: could not be loaded ({e}), skipped")
            continue
        ppl = None
        if not a.no_ppl:
            try:
                ppl = compute_perplexity(model, a.ppl_data, seq_len=min(a.seq_len, model.config.max_position_embeddings),
                                         max_tokens=a.ppl_tokens)
            except (FileNotFoundError, ValueError) as e:
                ppl = {"error": str(e)}
        matrix = {}
        for temp in temps:
            torch.manual_seed(a.seed)
            t0 = time.time()
            gens, records = [], []
            for pi, p in enumerate(prompts):
                samples = []
                for si in range(a.n_samples):
                    ts = time.time()
                    rec = generate_text(model, tok, p, details=True, max_new_tokens=a.max_tokens, temperature=temp,
                                        top_k=a.top_k, top_p=a.top_p, repetition_penalty=a.repetition_penalty)
                    samples.append(rec["continuation"])
                    records.append({"prompt_idx": pi, "sample_idx": si, "n_tokens": rec["n_tokens"], "stopped_by": rec["stopped_by"],
                                    "seconds": round(time.time() - ts, 3)})
                gens.append({"prompt": p, "samples": samples})
            out = {"run": run, "checkpoint": str(kw["checkpoint"]), **{k: v for k, v in meta.items() if v is not None},
                   "config": {"temperature": temp, "top_k": a.top_k, "top_p": a.top_p, "max_tokens": a.max_tokens,
                              "repetition_penalty": a.repetition_penalty, "n_samples": a.n_samples, "prompt_set": a.prompt_set,
                              "seed": a.seed},
                   "generations": gens, "samples": records, "generation_s": round(time.time() - t0, 2)}
            if ppl is not None:
                out["perplexity"] = ppl
            name = "generations.json" if len(temps) == 1 else f"generations_t{temp:g}.json"
            write_json(run_dir(a.output_dir, run) / name, out)
            n_tok = sum(r["n_tokens"] for r in records)
            matrix[f"{temp:g}"] = {"mean_tokens": n_tok / max(len(records), 1),
                                   "stopped_by": {w: sum(r["stopped_by"] == w for r in records) for w in ("eos", "max_tokens", "context")},
                                   "distinct_samples": len({s for g in gens for s in g["samples"]}) / max(len(records), 1),
                                   "tokens_per_second": round(n_tok / max(time.time() - t0, 1e-9), 1)}
            done.append(out)
            print(f"{run}: {len(gens)} prompts x {a.n_samples} samples at T={temp:g} -> {run_dir(a.output_dir, run) / name}"
                  + (f" (ppl {ppl['perplexity']:.2f})" if isinstance(ppl, dict) and "perplexity" in ppl else ""))
        if len(temps) > 1:
            write_json(run_dir(a.output_dir, run) / "temperature_matrix.json", {"run": run, "temperatures": matrix})
            # the default temperature's file doubles as generations.json for the tracks downstream
            base = min(temps, key=lambda t: abs(t - a.temperature))
            write_json(run_dir(a.output_dir, run) / "generations.json",
                       next(d for d in done if d["run"] == run and d["config"]["temperature"] == base))
        del model
    if a.combined and len({d["run"] for d in done}) > 1:
        names = list(dict.fromkeys(d["run"] for d in done))
        path = run_dir(a.output_dir, "_vs_".join(names[:3])) / "generations.json"
        write_json(path, {"config": done[0]["config"], "runs": done})
        print(f"combined -> {path}")
    if a.output and done:
        write_json(Path(a.output), done[-1] if len({d["run"] for d in done}) == 1 else {"config": done[0]["config"], "runs": done})
        print(f"-> {a.output}")


if __name__ == "__main__":
    main()
