#!/usr/bin/env python
"""Concept-geometry statistics (track 6b) on the arrays of ``extract_concept_geometry.py``.  Every
structural metric comes with a null: a permutation null (``--n-perm`` relabellings of the items) or,
for direction statistics, the closed form for random directions in D dimensions.

  cyclic      Mantel test (Spearman's rho) between activation distances and circular item distances, share
              of items whose nearest neighbours are their cyclic neighbours, and the winding of the
              items in the plane of the two leading principal components
  ordinal     Mantel correlation with |i - j|, k-NN overlap with the ordinal neighbours, and the
              Spearman correlation of the first principal component with the item order
  geographic  Mantel correlation with great-circle distances and the Procrustes fit of the two leading
              principal components onto (longitude, latitude)
  paired      consistency of the a -> b difference vectors over the pairs (mean pairwise cosine, z-score
              against random directions) and accuracy of completing b from a by the mean difference
  direction   consistency of the step vectors x[i+1] - x[i] of ordered sets, with its z-score
  smoothness  how far the centroid geometry moves between consecutive layers (distance-matrix
              correlation layer l vs l + 1): where structure forms, and where it is rewritten
  template    sensitivity: distance-matrix correlation between templates and the mean cosine distance
              of one item across templates
  subspace    participation ratio of the concept centroids, variance in the top-2 PCs, PC1 / PC2 ratio
  spectral    spectral entropy of the centroid covariance (nats, and normalised by its maximum)

    python tools/analysis/analyze_concept_geometry.py --input analysis/run/concept_geometry
    python tools/analysis/analyze_concept_geometry.py --input ... --only cyclic,ordinal --view pooled --n-perm 1000

``--view`` picks the activations: ``acts`` (item's last token, default), ``pooled`` (mean over the item's tokens) or
``last_tok`` (last token of the sentence).  Writes ``analysis.json`` next to the arrays (``analysis_<view>.json`` for
the other views).  CPU only.  Counterpart of the reference's ``scripts/analysis/analyze_concept_geometry.py``.
"""
from __future__ import annotations

import argparse
import json
import math
from pathlib import Path
from typing import Any, Optional

import numpy as np
from _common import write_json

ANALYSES = ["cyclic", "ordinal", "geographic", "paired", "direction", "smoothness", "template", "subspace", "spectral"]


# ------------------------------------------------------------------------------ distances and nulls
def pdist(x: np.ndarray) -> np.ndarray:
    g = x @ x.T
    n = np.diag(g)
    return np.sqrt(np.maximum(n[:, None] + n[None, :] - 2 * g, 0.0))


def upper(m: np.ndarray) -> np.ndarray:
    return m[np.triu_indices_from(m, 1)]


def corr(a: np.ndarray, b: np.ndarray) -> float:
    if a.std() < 1e-12 or b.std() < 1e-12:
        return 0.0
    return float(np.corrcoef(a, b)[0, 1])


def rank_avg(x: np.ndarray) -> np.ndarray:
    """Ranks 0..n-1 with ties sharing their average rank (what Spearman's rho is defined on)."""
    _, inv, cnt = np.unique(x, return_inverse=True, return_counts=True)
    last = np.cumsum(cnt) - 1.0
    return (last - (cnt - 1) / 2.0)[inv]


def mantel(da: np.ndarray, db: np.ndarray, n_perm: int, rng: np.random.Generator) -> dict:
    """Mantel test: Spearman's rho between the upper triangles of two distance matrices (rank correlation, as in
    the reference's ``mantel_test``: distances in activation space need not be linear in the target distance), with
    the items of one matrix relabelled for the null.  ``pearson_r`` is reported beside it."""
    a, b = upper(da), upper(db)
    iu = np.triu_indices_from(da, 1)
    ranks = np.zeros_like(da, dtype=float)
    ranks[iu] = rank_avg(a)
    ranks = ranks + ranks.T                               # a relabelled matrix has the same values, hence the same ranks
    rb = rank_avg(b)
    r = corr(ranks[iu], rb)
    n = da.shape[0]
    null = np.empty(n_perm)
    for i in range(n_perm):
        p = rng.permutation(n)
        null[i] = corr(ranks[np.ix_(p, p)][iu], rb)
    sd = float(null.std()) if n_perm else 0.0
    return {"r": r, "pearson_r": corr(a, b), "p": float(((null >= r).sum() + 1) / (n_perm + 1)),
            "null_mean": float(null.mean()) if n_perm else 0.0, "z": float((r - null.mean()) / sd) if sd > 1e-12 else 0.0}


def target_dist(n: int, cyclic: bool) -> np.ndarray:
    i = np.arange(n)
    d = np.abs(i[:, None] - i[None, :]).astype(float)
    return np.minimum(d, n - d) if cyclic else d


def haversine(coords: np.ndarray) -> np.ndarray:
    """Great-circle distances (km) between (lat, lon) rows in degrees."""
    lat, lon = np.radians(coords[:, 0]), np.radians(coords[:, 1])
    dlat, dlon = lat[:, None] - lat[None, :], lon[:, None] - lon[None, :]
    h = np.sin(dlat / 2) ** 2 + np.cos(lat)[:, None] * np.cos(lat)[None, :] * np.sin(dlon / 2) ** 2
    return 2 * 6371.0 * np.arcsin(np.sqrt(np.clip(h, 0.0, 1.0)))


def knn_overlap(d: np.ndarray, target: np.ndarray, k: int = 2) -> float:
    n = d.shape[0]
    hits = 0
    for i in range(n):
        a = set(np.argsort(d[i] + np.eye(n)[i] * 1e9)[:k])
        b = set(np.argsort(target[i] + np.eye(n)[i] * 1e9, kind="stable")[:k])
        hits += len(a & b)
    return hits / (n * k)


def knn_cyclic_hit(d: np.ndarray, k: int = 1) -> float:
    """Share of items with a cyclic neighbour ((i - 1) mod n or (i + 1) mod n) among their ``k`` nearest items."""
    n = d.shape[0]
    hits = 0
    for i in range(n):
        row = d[i].copy()
        row[i] = np.inf
        hits += bool({(i - 1) % n, (i + 1) % n} & set(np.argsort(row)[:k].tolist()))
    return hits / n


def knn_ordinal_window(d: np.ndarray, k: int = 3, window: int = 2) -> float:
    """Mean share of an item's ``k`` nearest items that lie within ``window`` positions of it in the order."""
    n = d.shape[0]
    total = 0.0
    for i in range(n):
        row = d[i].copy()
        row[i] = np.inf
        near = set(np.argsort(row)[:k].tolist())
        expected = {j for j in range(max(0, i - window), min(n, i + window + 1)) if j != i}
        total += len(near & expected) / min(k, len(expected)) if expected else 0.0
    return total / n


def knn_null(target: np.ndarray, k: int, n_perm: int, rng: np.random.Generator) -> float:
    """Expected k-NN overlap when the items are relabelled at random."""
    n = target.shape[0]
    if not n_perm:
        return k / max(n - 1, 1)
    vals = []
    for _ in range(min(n_perm, 200)):
        p = rng.permutation(n)
        vals.append(knn_overlap(target[np.ix_(p, p)], target, k))
    return float(np.mean(vals))


def spearman(a: np.ndarray, b: np.ndarray) -> float:
    ra, rb = np.argsort(np.argsort(a)).astype(float), np.argsort(np.argsort(b)).astype(float)
    return corr(ra, rb)


def pcs(x: np.ndarray, k: int = 2) -> tuple[np.ndarray, np.ndarray]:
    """Scores on the leading ``k`` principal components and all squared singular values."""
    xc = x - x.mean(0, keepdims=True)
    _, s, vt = np.linalg.svd(xc, full_matrices=False)
    return xc @ vt[:k].T, s ** 2


def cosine_consistency(v: np.ndarray) -> dict:
    """Mean pairwise cosine of the rows of ``v`` and its z-score against random directions: for unit vectors
    drawn uniformly in D dimensions a cosine has mean 0 and variance 1/D, the mean of m of them 1/(D m)."""
    m, D = v.shape
    if m < 2:
        return {"mean_cosine": float("nan"), "z": 0.0}
    u = v / (np.linalg.norm(v, axis=1, keepdims=True) + 1e-12)
    c = upper(u @ u.T)
    return {"mean_cosine": float(c.mean()), "z": float(c.mean() * math.sqrt(D * len(c)))}


# ------------------------------------------------------------------------------ per-kind analyses (one layer)
def analyse_cyclic(x: np.ndarray, n_perm: int, rng: np.random.Generator) -> dict:
    n = len(x)
    tgt = target_dist(n, True)
    d = pdist(x - x.mean(0))
    xy, _ = pcs(x, 2)
    ang = np.unwrap(np.arctan2(xy[:, 1], xy[:, 0]).tolist() + [math.atan2(xy[0, 1], xy[0, 0])])
    # items on a circle in order turn by +-2 pi in total; anything else gives a winding far from +-1
    winding = float((ang[-1] - ang[0]) / (2 * math.pi)) if xy.shape[1] == 2 else 0.0
    return {**mantel(d, tgt, n_perm, rng), "knn_overlap": knn_overlap(d, tgt), "knn_null": knn_null(tgt, 2, n_perm, rng),
            "knn_cyclic_hit": knn_cyclic_hit(d), "winding": winding}


def analyse_ordinal(x: np.ndarray, n_perm: int, rng: np.random.Generator) -> dict:
    n = len(x)
    tgt = target_dist(n, False)
    d = pdist(x - x.mean(0))
    xy, _ = pcs(x, 1)
    return {**mantel(d, tgt, n_perm, rng), "knn_overlap": knn_overlap(d, tgt), "knn_null": knn_null(tgt, 2, n_perm, rng),
            "knn_ordinal_window": knn_ordinal_window(d), "pc1_rank_correlation": abs(spearman(xy[:, 0], np.arange(n)))}


def analyse_geographic(x: np.ndarray, coords: np.ndarray, n_perm: int, rng: np.random.Generator) -> dict:
    d = pdist(x - x.mean(0))
    out = mantel(d, haversine(coords), n_perm, rng)
    # Procrustes fit of the PC plane onto (lon, lat): rotation / reflection + scale; 1 - residual = variance explained
    xy, _ = pcs(x, 2)
    g = np.stack([coords[:, 1], coords[:, 0]], 1)
    g = g - g.mean(0)
    a = xy / max(np.linalg.norm(xy), 1e-12)
    b = g / max(np.linalg.norm(g), 1e-12)
    s = np.linalg.svd(a.T @ b, compute_uv=False)
    out["map_fit"] = float(min(1.0, s.sum() ** 2))
    return out


def analyse_paired(x: np.ndarray) -> dict:
    a, b = x[0::2], x[1::2]
    diff = b - a
    out = cosine_consistency(diff)
    # leave-one-out completion: b_i predicted as a_i + mean of the other pairs' differences, nearest item wins
    m = len(diff)
    hits = 0
    for i in range(m):
        guess = a[i] + (diff.sum(0) - diff[i]) / max(m - 1, 1)
        dist = np.linalg.norm(x - guess, axis=1)
        dist[2 * i] = np.inf                                 # the query itself is not an answer
        hits += int(np.argmin(dist) == 2 * i + 1)
    out["completion_accuracy"] = hits / m
    out["completion_chance"] = 1.0 / max(len(x) - 1, 1)
    return out


def analyse_subspace(x: np.ndarray) -> dict:
    _, s = pcs(x, 1)
    tot = max(s.sum(), 1e-12)
    return {"participation_ratio": float(s.sum() ** 2 / max((s ** 2).sum(), 1e-12)), "top2_variance": float(s[:2].sum() / tot),
            "pc1_pc2_ratio": float(s[0] / max(s[1], 1e-12)) if len(s) > 1 else float("inf")}


def analyse_spectral(x: np.ndarray) -> dict:
    _, s = pcs(x, 1)
    p = s / max(s.sum(), 1e-12)
    h = float(-(p * np.log(p + 1e-12)).sum())
    return {"entropy": h, "normalised": h / math.log(max(len(s), 2))}


def analyse_template(acts: np.ndarray, l: int) -> dict:
    T = acts.shape[0]
    ds = [upper(pdist(acts[t, :, l] - acts[t, :, l].mean(0))) for t in range(T)]
    agree = [corr(ds[i], ds[j]) for i in range(T) for j in range(i + 1, T)]
    u = acts[:, :, l] / (np.linalg.norm(acts[:, :, l], axis=-1, keepdims=True) + 1e-12)     # [T, items, D]
    cosd = [1.0 - float((u[i] * u[j]).sum(-1).mean()) for i in range(T) for j in range(i + 1, T)]
    return {"distance_agreement": float(np.mean(agree)), "mean_cosine_distance": float(np.mean(cosd))}


# ------------------------------------------------------------------------------ one concept set
def analyse_set(acts: np.ndarray, info: dict, only: list[str], n_perm: int, rng: np.random.Generator) -> dict:
    T, n, L, D = acts.shape
    kind = info["kind"]
    out: dict[str, Any] = {"items": n, "layers": L, "templates": T}
    cent = acts.mean(0)                                          # [items, layers, D]: template-averaged
    coords = np.asarray(info["coordinates"], dtype=float) if kind == "geographic" and "coordinates" in info else None
    per_layer = []
    for l in range(L):
        x = cent[:, l].astype(np.float64)
        row: dict[str, Any] = {"layer": l}
        if kind == "cyclic" and "cyclic" in only:
            row["cyclic"] = analyse_cyclic(x, n_perm, rng)
        if kind == "ordinal" and "ordinal" in only:
            row["ordinal"] = analyse_ordinal(x, n_perm, rng)
        if coords is not None and "geographic" in only:
            row["geographic"] = analyse_geographic(x, coords, n_perm, rng)
        if kind == "paired" and "paired" in only:
            row["paired"] = analyse_paired(x)
        if kind in ("cyclic", "ordinal") and "direction" in only:
            steps = np.diff(x, axis=0)
            row["direction"] = cosine_consistency(steps)
            row["direction_consistency"] = row["direction"]["mean_cosine"]
        if "subspace" in only:
            row["subspace"] = analyse_subspace(x)
        if "spectral" in only:
            row["spectral"] = analyse_spectral(x)
        if "template" in only and T > 1:
            row["template"] = analyse_template(acts.astype(np.float64), l)
            row["template_agreement"] = row["template"]["distance_agreement"]
        per_layer.append(row)
    if "smoothness" in only and L > 1:
        dm = [upper(pdist(cent[:, l].astype(np.float64) - cent[:, l].mean(0))) for l in range(L)]
        for l in range(L - 1):
            per_layer[l]["smoothness_to_next"] = corr(dm[l], dm[l + 1])
        out["smoothness"] = {"mean": float(np.mean([per_layer[l]["smoothness_to_next"] for l in range(L - 1)])),
                             "least_smooth_layer": int(np.argmin([per_layer[l]["smoothness_to_next"] for l in range(L - 1)]))}
    out["per_layer"] = per_layer
    main_key = {"cyclic": "cyclic", "ordinal": "ordinal", "geographic": "geographic"}.get(kind)
    if main_key and main_key in only and main_key in per_layer[0]:
        best = max(per_layer, key=lambda r: r[main_key]["r"])
        out["best_layer"] = {"layer": best["layer"], **best[main_key]}
        sig = [r["layer"] for r in per_layer if r[main_key]["p"] < 0.05]
        out["first_significant_layer"] = sig[0] if sig else None         # where the structure emerges
        out["significant_layers"] = len(sig)
    if kind == "paired" and "paired" in only:
        best = max(per_layer, key=lambda r: r["paired"]["completion_accuracy"])
        out["best_layer"] = {"layer": best["layer"], **best["paired"]}
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True, help="a run's concept_geometry directory")
    ap.add_argument("--only", default=",".join(ANALYSES))
    ap.add_argument("--concept-sets", default=None)
    ap.add_argument("--view", default="acts", choices=["acts", "pooled", "last_tok"])
    ap.add_argument("--n-perm", type=int, default=200)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--output", default=None)
    a = ap.parse_args()
    only = [s.strip() for s in a.only.split(",")]
    # earlier names of two analyses
    only = ["template" if s == "template_sensitivity" else "subspace" if s == "subspace_diagnostics" else s for s in only]
    unknown = set(only) - set(ANALYSES)
    if unknown:
        raise SystemExit(f"unknown analyses {sorted(unknown)}; choose from {ANALYSES}")
    d = Path(a.input)
    meta = json.loads((d / "meta.json").read_text())
    rng = np.random.default_rng(a.seed)
    wanted: Optional[set[str]] = {s.strip() for s in a.concept_sets.split(",")} if a.concept_sets else None
    res: dict[str, Any] = {"run": meta.get("run"), "n_perm": a.n_perm, "view": a.view, "analyses": only, "sets": {}}
    for name, info in meta["sets"].items():
        if wanted is not None and name not in wanted:
            continue
        with np.load(d / f"{name}.npz") as z:
            acts = z[a.view] if a.view in z.files else z["acts"]
        res["sets"][name] = {"kind": info["kind"], "tier": info.get("tier", 1), **analyse_set(acts, info, only, a.n_perm, rng)}
    # one line per set: the headline statistic at its best layer
    summary = {}
    for name, s in res["sets"].items():
        b = s.get("best_layer")
        if b:
            key = "r" if "r" in b else "completion_accuracy"
            summary[name] = {"kind": s["kind"], "layer": b["layer"], key: b[key], **({"p": b["p"]} if "p" in b else {})}
    res["summary"] = summary
    out = Path(a.output) if a.output else d / ("analysis.json" if a.view == "acts" else f"analysis_{a.view}.json")
    write_json(out, res)
    for name, s in summary.items():
        stat = f"r = {s['r']:.3f} (p = {s['p']:.3f})" if "r" in s else f"completion {s['completion_accuracy']:.2f}"
        print(f"  {name:14s} {s['kind']:11s} best layer {s['layer']:3d}  {stat}")
    print(f"{len(res['sets'])} concept sets -> {out}")


if __name__ == "__main__":
    main()
