#!/usr/bin/env python
"""Plots for the concept-geometry track (6c) from the arrays of ``extract_concept_geometry.py`` and the
statistics of ``analyze_concept_geometry.py``:

  * per set: PCA-2 of the concept centroids at the set's best layer (items joined in order for cyclic
    and ordinal sets, pairs joined by arrows for paired sets, the PC plane rotated onto the map for
    geographic sets, with the true positions drawn faintly)
  * per set: the headline statistic over depth (Mantel r with its permutation-null mean; completion
    accuracy for paired sets) and the layer-to-layer smoothness
  * all sets: a layer x set heat map of the headline statistic and a table of best layers

With matplotlib the figures are PNG files; without it the same figures are drawn as SVG by the built-in plotting
layer (``kotodama_b200/eval/plot_utils.py``), and the coordinates (``<set>_pca2.csv``) and per-layer curves
(``curves.csv``) are written as well.

    python tools/analysis/visualize_concept_geometry.py --input analysis/run/concept_geometry [--view pooled]

Counterpart of the reference's ``scripts/analysis/visualize_concept_geometry.py``.
"""
from __future__ import annotations

import argparse
import csv
import json
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[2]))
from kotodama_b200.eval import plot_utils as pu  # noqa: E402

HEADLINE = {"cyclic": ("cyclic", "r"), "ordinal": ("ordinal", "r"), "geographic": ("geographic", "r"),
            "paired": ("paired", "completion_accuracy")}


def headline_curve(s: dict) -> tuple[list[float], list[float]]:
    """The set's headline statistic per layer and, where there is one, the null mean per layer."""
    key = HEADLINE.get(s["kind"])
    if not key:
        return [], []
    rows = [r[key[0]] for r in s["per_layer"] if key[0] in r]
    null = [r.get("null_mean", r.get("completion_chance", 0.0)) for r in rows]
    return [r[key[1]] for r in rows], null


def plane(x: np.ndarray) -> np.ndarray:
    xc = x - x.mean(0)
    _, _, vt = np.linalg.svd(xc, full_matrices=False)
    return xc @ vt[:2].T


def onto_map(xy: np.ndarray, coords: np.ndarray) -> np.ndarray:
    """Rotate / reflect / scale the PC plane onto (lon, lat) (orthogonal Procrustes)."""
    g = np.stack([coords[:, 1], coords[:, 0]], 1)
    gm = g.mean(0)
    u, s, vt = np.linalg.svd(xy.T @ (g - gm))
    rot = u @ vt
    scale = s.sum() / max((xy ** 2).sum(), 1e-12)
    return xy @ rot * scale + gm


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    ap.add_argument("--view", default="acts", choices=["acts", "pooled", "last_tok"])
    ap.add_argument("--only", default=None, help="comma-separated concept sets to draw; default: all")
    ap.add_argument("--style", default="publication", help="'dark' switches the matplotlib figures to a dark background")
    a = ap.parse_args()
    only = {w.strip() for w in a.only.split(",")} if a.only else None
    d = Path(a.input)
    meta = json.loads((d / "meta.json").read_text())
    af = d / ("analysis.json" if a.view == "acts" else f"analysis_{a.view}.json")
    ana = json.loads(af.read_text()) if af.exists() else {"sets": {}}
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        pu.apply_style(plt, dark=a.style == "dark")
    except ImportError:
        plt = None
    curves: dict[str, list[float]] = {}
    for name, info in meta["sets"].items():
        if only is not None and name not in only:
            continue
        with np.load(d / f"{name}.npz") as z:
            acts = (z[a.view] if a.view in z.files else z["acts"]).mean(0)             # [items, layers, D]
        s = ana["sets"].get(name, {})
        layer = s.get("best_layer", {}).get("layer", acts.shape[1] - 1)
        xy = plane(acts[:, layer].astype(np.float64))
        kind = info["kind"]
        coords = np.asarray(info["coordinates"], dtype=float) if kind == "geographic" and "coordinates" in info else None
        if coords is not None:
            xy = onto_map(xy, coords)
        if s:
            c, null = headline_curve(s)
            if c:
                curves[name] = c
                curves[f"{name}|null"] = null
            sm = [r["smoothness_to_next"] for r in s["per_layer"] if "smoothness_to_next" in r]
            if sm:
                curves[f"{name}|smoothness"] = sm
        if plt is None:
            with open(d / f"{name}_pca2.csv", "w", newline="") as fh:
                w = csv.writer(fh)
                w.writerow(["item", "pc1", "pc2", "layer"])
                for it, p in zip(info["items"], xy):
                    w.writerow([it, float(p[0]), float(p[1]), layer])
            (d / f"{name}_pca2.svg").write_text(pu.scatter(
                xy, labels=info["items"], title=f"{name} ({kind}): layer {layer}",
                connect="loop" if kind == "cyclic" else "path" if kind == "ordinal" else "",
                arrows=[(i, i + 1) for i in range(0, len(xy) - 1, 2)] if kind == "paired" else None,
                ghosts=[(c[1], c[0]) for c in coords] if coords is not None else None))
            if name in curves:
                lines = {HEADLINE[kind][1]: curves[name], "null": curves[f"{name}|null"]}
                if f"{name}|smoothness" in curves:
                    lines["smoothness to next layer"] = curves[f"{name}|smoothness"]
                (d / f"{name}_depth.svg").write_text(pu.line_chart(lines, title=name, xlabel="layer (0 = embeddings)", dashed=["null"],
                                                                   colors={HEADLINE[kind][1]: "#1f77b4", "null": "#888888",
                                                                           "smoothness to next layer": "#2ca02c"}))
            continue
        fig, ax = plt.subplots(figsize=(4.8, 4.8))
        if kind in ("cyclic", "ordinal"):
            path = np.vstack([xy, xy[:1]]) if kind == "cyclic" else xy
            ax.plot(*path.T, "-", lw=0.6, alpha=0.5)
        if kind == "paired":
            for i in range(0, len(xy) - 1, 2):
                ax.annotate("", xy=xy[i + 1], xytext=xy[i], arrowprops={"arrowstyle": "->", "lw": 0.7, "alpha": 0.6})
        if coords is not None:
            ax.scatter(coords[:, 1], coords[:, 0], s=10, c="lightgray", label="true position")
            for p, q in zip(xy, coords):
                ax.plot([p[0], q[1]], [p[1], q[0]], lw=0.4, c="lightgray")
            ax.legend(fontsize=6)
        ax.scatter(*xy.T, s=18, c=np.arange(len(xy)), cmap="twilight" if kind == "cyclic" else "viridis")
        for it, p in zip(info["items"], xy):
            ax.annotate(it, p, fontsize=7)
        ax.set_title(f"{name} ({kind}): layer {layer}")
        fig.tight_layout()
        fig.savefig(d / f"{name}_pca2.png", dpi=120)
        plt.close(fig)
        if name in curves:
            fig, ax = plt.subplots(figsize=(5, 3))
            ax.plot(curves[name], marker="o", ms=3, label=HEADLINE[kind][1])
            ax.plot(curves[f"{name}|null"], ls="--", lw=0.8, label="null")
            if f"{name}|smoothness" in curves:
                ax.plot(curves[f"{name}|smoothness"], lw=0.8, alpha=0.7, label="smoothness to next layer")
            ax.set_xlabel("layer (0 = embeddings)")
            ax.set_title(name)
            ax.legend(fontsize=6)
            fig.tight_layout()
            fig.savefig(d / f"{name}_depth.png", dpi=120)
            plt.close(fig)
    main_curves = {k: v for k, v in curves.items() if "|" not in k}
    if plt is None:
        with open(d / "curves.csv", "w", newline="") as fh:
            w = csv.writer(fh)
            for k, v in curves.items():
                w.writerow([k] + list(v))
        if main_curves:
            names = list(main_curves)
            (d / "overview.svg").write_text(pu.heatmap([main_curves[n] for n in names], title="headline statistic over depth",
                                                       xlabel="layer", row_labels=names, vmax=1.0))
    elif main_curves:
        names = list(main_curves)
        m = np.array([main_curves[n] for n in names])
        fig, ax = plt.subplots(figsize=(0.35 * m.shape[1] + 2.5, 0.3 * len(names) + 1.5))
        im = ax.imshow(m, aspect="auto", cmap="viridis", vmin=min(0.0, float(m.min())), vmax=1.0)
        ax.set_yticks(range(len(names)))
        ax.set_yticklabels(names, fontsize=7)
        ax.set_xlabel("layer")
        ax.set_title("headline statistic over depth")
        fig.colorbar(im)
        fig.tight_layout()
        fig.savefig(d / "overview.png", dpi=120)
        plt.close(fig)
    print(f"{'plots' if plt else 'SVG figures and CSV (matplotlib is not installed)'} -> {d}")


if __name__ == "__main__":
    main()
