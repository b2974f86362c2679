#!/usr/bin/env python
"""Plots for the activation-geometry track (5b) from the files written by
``extract_activation_geometry.py``: per-layer RankMe / participation ratio, trajectory norms,
head entropy, PCA point clouds.  Needs matplotlib; without it the script writes the same
series as CSV so they can be plotted elsewhere.

    python tools/analysis/visualize_activation_geometry.py --run my-run [--output-dir analysis]

Counterpart of the reference's ``scripts/analysis/visualize_activation_geometry.py``.
"""
from __future__ import annotations

import argparse
import csv
import json
from pathlib import Path

import numpy as np


def series(geo: dict) -> dict[str, list[float]]:
    s: dict[str, list[float]] = {}
    if "eigenspectra" in geo:
        s["rankme"] = [e["rankme"] for e in geo["eigenspectra"]]
        s["participation_ratio"] = [e["participation_ratio"] for e in geo["eigenspectra"]]
    if "trajectories" in geo:
        s["mean_norm"] = geo["trajectories"]["mean_norm_per_layer"]
        s["step_cosine"] = geo["trajectories"]["mean_step_cosine"]
    for l, a in geo.get("attention", {}).items():
        s[f"head_entropy_layer{l}"] = a["head_entropy"]
    return s


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--run", required=True)
    ap.add_argument("--output-dir", default="analysis")
    a = ap.parse_args()
    d = Path(a.output_dir) / a.run / "activation_geometry"
    geo = json.loads((d / "geometry.json").read_text())
    s = series(geo)
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
    except ImportError:
        with open(d / "series.csv", "w", newline="") as fh:
            w = csv.writer(fh)
            for k, v in s.items():
                w.writerow([k] + list(v))
        print(f"matplotlib is not installed: wrote {d / 'series.csv'}")
        return
    for k, v in s.items():
        fig, ax = plt.subplots(figsize=(5, 3))
        ax.plot(v, marker="o", ms=3)
        ax.set_title(f"{a.run}: {k}")
        ax.set_xlabel("head" if k.startswith("head_entropy") else "layer")
        fig.tight_layout()
        fig.savefig(d / f"{k}.png", dpi=120)
        plt.close(fig)
    npz = d / "arrays.npz"
    if npz.exists():
        pc = np.load(npz).get("point_clouds")
        if pc is not None:
            for l in sorted({0, len(pc) // 2, len(pc) - 1}):
                fig = plt.figure(figsize=(4, 4))
                ax = fig.add_subplot(projection="3d")
                ax.scatter(pc[l][:, 0], pc[l][:, 1], pc[l][:, 2], s=12)
                ax.set_title(f"{a.run}: PCA-3, layer {l}")
                fig.savefig(d / f"point_cloud_layer{l}.png", dpi=120)
                plt.close(fig)
    print(f"plots -> {d}")


if __name__ == "__main__":
    main()
