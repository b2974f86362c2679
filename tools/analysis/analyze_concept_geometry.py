#!/usr/bin/env python
"""Concept-geometry statistics (track 6b) on the arrays of ``extract_concept_geometry.py``; every
metric comes with a permutation null (``--n-perm``):

  cyclic     Mantel correlation between activation distances and circular item distances, and the
             share of items whose nearest neighbours are their cyclic neighbours
  ordinal    Mantel correlation with |i - j| and k-NN overlap with the ordinal neighbours
  direction  consistency of the step vectors x[i+1] - x[i] (mean pairwise cosine)
  template   sensitivity: distance-matrix correlation between templates
  subspace   participation ratio of the concept centroids and variance in the top-2 PCs

    python tools/analysis/analyze_concept_geometry.py --input analysis/run/concept_geometry [--only cyclic,ordinal]

CPU only.  Counterpart of the reference's ``scripts/analysis/analyze_concept_geometry.py``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import numpy as np
from _common import write_json

ANALYSES = ["cyclic", "ordinal", "direction", "template", "subspace"]


def pdist(x: np.ndarray) -> np.ndarray:
    g = x @ x.T
    n = np.diag(g)
    return np.sqrt(np.maximum(n[:, None] + n[None, :] - 2 * g, 0.0))


def upper(m: np.ndarray) -> np.ndarray:
    return m[np.triu_indices_from(m, 1)]


def mantel(da: np.ndarray, db: np.ndarray, n_perm: int, rng: np.random.Generator) -> dict:
    a, b = upper(da), upper(db)
    r = float(np.corrcoef(a, b)[0, 1])
    n = da.shape[0]
    null = []
    for _ in range(n_perm):
        p = rng.permutation(n)
        null.append(np.corrcoef(upper(da[np.ix_(p, p)]), b)[0, 1])
    null = np.asarray(null)
    return {"r": r, "p": float(((null >= r).sum() + 1) / (n_perm + 1)), "null_mean": float(null.mean())}


def target_dist(n: int, cyclic: bool) -> np.ndarray:
    i = np.arange(n)
    d = np.abs(i[:, None] - i[None, :]).astype(float)
    return np.minimum(d, n - d) if cyclic else d


def knn_overlap(d: np.ndarray, target: np.ndarray, k: int = 2) -> float:
    n = d.shape[0]
    hits = 0
    for i in range(n):
        a = set(np.argsort(d[i] + np.eye(n)[i] * 1e9)[:k])
        b = set(np.argsort(target[i] + np.eye(n)[i] * 1e9, kind="stable")[:k])
        hits += len(a & b)
    return hits / (n * k)


def analyse_set(acts: np.ndarray, kind: str, only: list[str], n_perm: int, rng: np.random.Generator) -> dict:
    T, n, L, D = acts.shape
    out: dict = {"items": n, "layers": L}
    cent = acts.mean(0)                                          # [items, layers, D]
    per_layer = []
    for l in range(L):
        x = cent[:, l]
        d = pdist(x - x.mean(0))
        row: dict = {"layer": l}
        if kind in ("cyclic", "ordinal") and kind in only:
            tgt = target_dist(n, kind == "cyclic")
            row[kind] = {**mantel(d, tgt, n_perm, rng), "knn_overlap": knn_overlap(d, tgt)}
        if kind in ("cyclic", "ordinal") and "direction" in only:
            steps = np.diff(x, axis=0)
            steps = steps / (np.linalg.norm(steps, axis=1, keepdims=True) + 1e-9)
            c = steps @ steps.T
            row["direction_consistency"] = float(upper(c).mean())
        if "subspace" in only:
            xc = x - x.mean(0)
            s = np.linalg.svd(xc, compute_uv=False) ** 2
            row["subspace"] = {"participation_ratio": float(s.sum() ** 2 / max((s ** 2).sum(), 1e-12)),
                               "top2_variance": float(s[:2].sum() / max(s.sum(), 1e-12))}
        if "template" in only and T > 1:
            ds = [upper(pdist(acts[t, :, l] - acts[t, :, l].mean(0))) for t in range(T)]
            cs = [np.corrcoef(ds[i], ds[j])[0, 1] for i in range(T) for j in range(i + 1, T)]
            row["template_agreement"] = float(np.mean(cs))
        per_layer.append(row)
    out["per_layer"] = per_layer
    if kind in ("cyclic", "ordinal") and kind in only:
        best = max(per_layer, key=lambda r: r[kind]["r"])
        out["best_layer"] = {"layer": best["layer"], **best[kind]}
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--only", default=",".join(ANALYSES))
    ap.add_argument("--n-perm", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args()
    only = [s.strip() for s in a.only.split(",")]
    d = Path(a.input)
    meta = json.loads((d / "meta.json").read_text())
    rng = np.random.default_rng(a.seed)
    res = {"run": meta.get("run"), "n_perm": a.n_perm, "sets": {}}
    for name, info in meta["sets"].items():
        acts = np.load(d / f"{name}.npz")["acts"]
        res["sets"][name] = {"kind": info["kind"], **analyse_set(acts, info["kind"], only, a.n_perm, rng)}
    write_json(d / "analysis.json", res)
    print(f"{len(res['sets'])} concept sets -> {d / 'analysis.json'}")


if __name__ == "__main__":
    main()
