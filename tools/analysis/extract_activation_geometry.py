#!/usr/bin/env python
"""Activation-geometry extraction (track 5a): geometric objects of a checkpoint's residual stream.

Components (``--components``, comma separated; default all):
  point_clouds    PCA-3 projection of last-token states per layer over a prompt set
  eigenspectra    covariance eigenvalues of the per-layer token states (participation ratio, RankMe)
  trajectories    layer-to-layer path of each prompt's last-token state (norms, step cosines)
  attention       mean attention-distance and per-head entropy of selected layers
  effective_rank  stable rank and entropy rank of every projection matrix (weights only, CPU)
  procrustes      orthogonal-Procrustes distance between the layer states of two checkpoints

    python tools/analysis/extract_activation_geometry.py --checkpoint ckpt.pt --name run --device cuda
    python tools/analysis/extract_activation_geometry.py --checkpoints a,b --components procrustes

Writes ``<output-dir>/<run>/activation_geometry/{geometry.json, arrays.npz}``.  Counterpart of the
reference's ``scripts/analysis/extract_activation_geometry.py``.
"""
from __future__ import annotations

import argparse
import math

import numpy as np
import torch
from _common import ROOT, add_checkpoint_args, load_yaml, open_model, run_dir, select_checkpoints, tokenizer, write_json

from kotodama_b200.eval import forward_with_states

ALL = ["point_clouds", "eigenspectra", "trajectories", "attention", "effective_rank", "procrustes"]


def spectrum_stats(x: np.ndarray) -> dict:
    x = x - x.mean(0, keepdims=True)
    s = np.linalg.svd(x, compute_uv=False) ** 2
    p = s / max(s.sum(), 1e-12)
    return {"participation_ratio": float(s.sum() ** 2 / max((s ** 2).sum(), 1e-12)),
            "rankme": float(math.exp(-(p * np.log(p + 1e-12)).sum())), "top": s[:16].tolist()}


def pca3(x: np.ndarray) -> np.ndarray:
    x = x - x.mean(0, keepdims=True)
    _, _, vt = np.linalg.svd(x, full_matrices=False)
    return x @ vt[:3].T


def collect_states(model, tok, prompts, device, attn_layers):
    last, toks, attn = [], [], {}
    for p in prompts:
        ids = torch.tensor([tok.encode(p)[: model.config.max_position_embeddings]], device=device)
        res = forward_with_states(model, ids, attention_layers=attn_layers)
        last.append(torch.stack([s[0, -1].float().cpu() for s in res.states]).numpy())      # [L+1, D]
        toks.append(torch.stack([s[0].float().cpu() for s in res.states]).numpy())            # [L+1, T, D]
        for l, a in res.attention.items():
            attn.setdefault(l, []).append(a[0].float().cpu().numpy())                          # [H, T, T]
    return np.stack(last), toks, attn


def weight_ranks(model) -> dict:
    out = {}
    for name, p in model.named_parameters():
        if p.ndim == 2 and "embed" not in name and "lm_head" not in name:
            s = torch.linalg.svdvals(p.detach().float().cpu())
            q = (s / s.sum()).numpy()
            out[name] = {"stable_rank": float((s ** 2).sum() / (s[0] ** 2)), "entropy_rank": float(math.exp(-(q * np.log(q + 1e-12)).sum()))}
    return out


def procrustes_distance(a: np.ndarray, b: np.ndarray) -> float:
    a = (a - a.mean(0)) / (np.linalg.norm(a - a.mean(0)) + 1e-12)
    b = (b - b.mean(0)) / (np.linalg.norm(b - b.mean(0)) + 1e-12)
    s = np.linalg.svd(a.T @ b, compute_uv=False)
    return float(max(0.0, 1.0 - s.sum() ** 2))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_checkpoint_args(ap)
    ap.add_argument("--components", default=",".join(ALL))
    ap.add_argument("--prompt-set", default="extended")
    ap.add_argument("--prompts-file", default=str(ROOT / "configs" / "prompts.yaml"))
    ap.add_argument("--attention-layers", default="0,-1")
    a = ap.parse_args()
    comps = [c.strip() for c in a.components.split(",") if c.strip()]
    unknown = set(comps) - set(ALL)
    if unknown:
        raise SystemExit(f"unknown components {sorted(unknown)}; choose from {ALL}")
    prompts = load_yaml(a.prompts_file)[a.prompt_set]
    tok = tokenizer(a.tokenizer)
    last_by_run = {}
    for run, kw in select_checkpoints(a):
        model, _ = open_model(kw, a.device)
        L = model.config.num_layers
        attn_layers = sorted({int(x) % L for x in a.attention_layers.split(",")}) if "attention" in comps else []
        out, arrays = {"run": run, "layers": L, "prompts": len(prompts)}, {}
        need_fwd = set(comps) & {"point_clouds", "eigenspectra", "trajectories", "attention", "procrustes"}
        if need_fwd:
            last, toks, attn = collect_states(model, tok, prompts, a.device, attn_layers)
            last_by_run[run] = last
        if "point_clouds" in comps:
            arrays["point_clouds"] = np.stack([pca3(last[:, l]) for l in range(L + 1)])                 # [L+1, P, 3]
        if "eigenspectra" in comps:
            out["eigenspectra"] = [spectrum_stats(np.concatenate([t[l] for t in toks])) for l in range(L + 1)]
        if "trajectories" in comps:
            norms = np.linalg.norm(last, axis=-1)                                                        # [P, L+1]
            d = np.diff(last, axis=1)
            cos = (d[:, 1:] * d[:, :-1]).sum(-1) / (np.linalg.norm(d[:, 1:], axis=-1) * np.linalg.norm(d[:, :-1], axis=-1) + 1e-9)
            out["trajectories"] = {"mean_norm_per_layer": norms.mean(0).tolist(), "mean_step_cosine": cos.mean(0).tolist()}
            arrays["trajectory_norms"] = norms
        if "attention" in comps:
            att = {}
            for l, mats in attn.items():
                ent, dist = [], []
                for m in mats:
                    T = m.shape[-1]
                    ent.append(-(m * np.log(m + 1e-12)).sum(-1).mean(-1))                                # [H]
                    idx = np.arange(T)
                    dist.append((m * np.abs(idx[:, None] - idx[None, :])).sum(-1).mean(-1))
                att[str(l)] = {"head_entropy": np.mean(ent, 0).tolist(), "mean_attention_distance": np.mean(dist, 0).tolist()}
            out["attention"] = att
        if "effective_rank" in comps:
            out["effective_rank"] = weight_ranks(model)
        d = run_dir(a.output_dir, run, "activation_geometry")
        write_json(d / "geometry.json", out)
        if arrays:
            np.savez_compressed(d / "arrays.npz", **arrays)
        print(f"{run}: {sorted(set(comps) - {'procrustes'})} -> {d}")
    if "procrustes" in comps and len(last_by_run) >= 2:
        names = list(last_by_run)
        res = {}
        for i, x in enumerate(names):
            for y in names[i + 1:]:
                A, B = last_by_run[x], last_by_run[y]
                n = min(A.shape[1], B.shape[1])
                res[f"{x}|{y}"] = [procrustes_distance(A[:, l], B[:, l]) for l in range(n)]
        write_json(run_dir(a.output_dir, "_pairs") / "procrustes.json", res)
        print(f"procrustes: {len(res)} pairs -> {run_dir(a.output_dir, '_pairs') / 'procrustes.json'}")


if __name__ == "__main__":
    main()
