#!/usr/bin/env python
"""Plots for the concept-geometry track: PCA-2 of the concept centroids at the best layer of each
set, and the per-layer Mantel curve.  Needs matplotlib; otherwise writes the coordinates as CSV.

    python tools/analysis/visualize_concept_geometry.py --input analysis/run/concept_geometry

Counterpart of the reference's ``scripts/analysis/visualize_concept_geometry.py``.
"""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path

import numpy as np


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True)
    a = ap.parse_args()
    d = Path(a.input)
    meta = json.loads((d / "meta.json").read_text())
    ana = json.loads((d / "analysis.json").read_text()) if (d / "analysis.json").exists() else {"sets": {}}
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        plt = None
    for name, info in meta["sets"].items():
        acts = np.load(d / f"{name}.npz")["acts"].mean(0)                 # [items, layers, D]
        layer = ana["sets"].get(name, {}).get("best_layer", {}).get("layer", acts.shape[1] - 1)
        x = acts[:, layer] - acts[:, layer].mean(0)
        _, _, vt = np.linalg.svd(x, full_matrices=False)
        xy = x @ vt[:2].T
        if plt is None:
            with open(d / f"{name}_pca2.csv", "w", newline="") as fh:
                w = csv.writer(fh)
                w.writerow(["item", "pc1", "pc2", "layer"])
                for it, p in zip(info["items"], xy):
                    w.writerow([it, float(p[0]), float(p[1]), layer])
            continue
        fig, ax = plt.subplots(figsize=(4.5, 4.5))
        ax.plot(*xy.T, "-", lw=0.6, alpha=0.5)
        ax.scatter(*xy.T, s=18)
        for it, p in zip(info["items"], xy):
            ax.annotate(it, p, fontsize=7)
        ax.set_title(f"{name}: layer {layer}")
        fig.tight_layout()
        fig.savefig(d / f"{name}_pca2.png", dpi=120)
        plt.close(fig)
    print(f"{'plots' if plt else 'CSV (matplotlib missing)'} -> {d}")


if __name__ == "__main__":
    main()
