#!/usr/bin/env python
"""Plots for the activation-geometry track (5b) from the files written by
``extract_activation_geometry.py``.

Per run (``--run``): per-layer RankMe / participation ratio of the states, trajectory norms, step
cosines and step lengths, head entropy (selected layers as curves, all layers as a layer x head map),
effective rank of every weight type over depth, TwoNN dimension of the token clouds, the share of the
attention branch in the state, PCA point clouds, and the saved attention matrices.  With ``--runs a,b``
the same series are overlaid for several runs and the Procrustes distances between them are drawn.

With matplotlib the figures are PNG files; without it the same figures are drawn as SVG by the built-in
plotting layer (``kotodama_b200/eval/plot_utils.py``) and the series are also written as CSV (``series.csv``,
``head_entropy_map.csv``), so the track produces pictures on a bare Python install.

    python tools/analysis/visualize_activation_geometry.py --run my-run [--output-dir analysis]
    python tools/analysis/visualize_activation_geometry.py --runs a,b [--output-dir analysis]

Counterpart of the reference's ``scripts/analysis/visualize_activation_geometry.py``.
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


def series(geo: dict) -> dict[str, list[float]]:
    """Every 1-D series of a run's ``geometry.json``, keyed by what it shows."""
    s: dict[str, list[float]] = {}
    if "eigenspectra" in geo:
        s["rankme"] = [e["rankme"] for e in geo["eigenspectra"]]
        s["participation_ratio"] = [e["participation_ratio"] for e in geo["eigenspectra"]]
    tr = geo.get("trajectories")
    if tr:
        s["mean_norm"] = tr["mean_norm_per_layer"]
        s["step_cosine"] = tr["mean_step_cosine"]
        if "mean_step_length" in tr:
            s["step_length"] = tr["mean_step_length"]
    for l, a in geo.get("attention", {}).items():
        s[f"head_entropy_layer{l}"] = a["head_entropy"]
        s[f"attention_distance_layer{l}"] = a["mean_attention_distance"]
    he = geo.get("head_entropy")
    if he:
        s["head_entropy_mean"] = he["mean_per_layer"]
        s["head_entropy_min"] = he["min_per_layer"]
    er = geo.get("effective_rank", {})
    for wtype, measures in er.items():
        if isinstance(measures, dict) and "participation_ratio" in measures:
            s[f"effective_rank_{wtype}"] = measures["participation_ratio"]
            s[f"stable_rank_{wtype}"] = measures["stable_rank"]
    for wtype, top in geo.get("weight_spectra", {}).items():
        s[f"top_singular_value_{wtype}"] = top
    ao = geo.get("attention_outputs")
    if ao:
        s["attention_branch_share"] = ao["branch_to_state_norm_ratio"]
        s["attention_branch_rankme"] = [e["rankme"] for e in ao["spectrum"]]
    tc = geo.get("topo_clouds", {}).get("twonn_dimension")
    if tc:
        s["twonn_dimension"] = [tc[k] for k in sorted(tc, key=int)]
    pc = geo.get("point_clouds", {}).get("spread_per_layer")
    if pc:
        s["point_cloud_spread"] = pc
    return s


def write_csv(path: Path, rows: dict[str, list[float]]) -> None:
    with open(path, "w", newline="") as fh:
        w = csv.writer(fh)
        for k, v in rows.items():
            w.writerow([k] + list(v))


def svg_run(d: Path, run: str, s: dict[str, list[float]]) -> int:
    """The per-run figures without matplotlib: one SVG per series, the PCA clouds, the head-entropy map."""
    n = 0
    for k, v in s.items():
        per_head = k.startswith(("head_entropy_layer", "attention_distance_layer"))
        (d / f"{k}.svg").write_text(pu.line_chart({run: v}, title=f"{run}: {k}", xlabel="head" if per_head else "layer"))
        n += 1
    npz = d / "arrays.npz"
    if npz.exists():
        with np.load(npz) as z:
            pc = z["point_clouds"] if "point_clouds" in z.files else None
        if pc is not None:
            for l in sorted({0, len(pc) // 2, len(pc) - 1}):
                (d / f"point_cloud_layer{l}.svg").write_text(
                    pu.scatter(pc[l][:, :2], title=f"{run}: PCA, layer {l}", xlabel="PC 1", ylabel="PC 2"))
                n += 1
    he = d / "head_entropy.npz"
    if he.exists():
        with np.load(he) as z:
            (d / "head_entropy_map.svg").write_text(
                pu.heatmap(z["entropy"].tolist(), title=f"{run}: attention entropy (nats)", xlabel="head", ylabel="layer"))
        n += 1
    return n


def load_run(output_dir: str, run: str) -> tuple[Path, dict]:
    d = Path(output_dir) / run / "activation_geometry"
    return d, json.loads((d / "geometry.json").read_text())


def plot_run(plt, d: Path, run: str, s: dict[str, list[float]]) -> None:
    for k, v in s.items():
        fig, ax = plt.subplots(figsize=(5, 3))
        ax.plot(v, marker="o", ms=3)
        ax.set_title(f"{run}: {k}")
        ax.set_xlabel("head" if k.startswith(("head_entropy_layer", "attention_distance_layer")) else "layer")
        fig.tight_layout()
        fig.savefig(d / f"{k}.png", dpi=120)
        plt.close(fig)
    npz = d / "arrays.npz"
    if npz.exists():
        with np.load(npz) as z:
            pc = z["point_clouds"] if "point_clouds" in z.files else None
        if pc is not None:
            for l in sorted({0, len(pc) // 2, len(pc) - 1}):
                fig = plt.figure(figsize=(4, 4))
                ax = fig.add_subplot(projection="3d")
                ax.scatter(pc[l][:, 0], pc[l][:, 1], pc[l][:, 2], s=12)
                ax.set_title(f"{run}: PCA-3, layer {l}")
                fig.savefig(d / f"point_cloud_layer{l}.png", dpi=120)
                plt.close(fig)
    he = d / "head_entropy.npz"
    if he.exists():
        with np.load(he) as z:
            m = z["entropy"]
        fig, ax = plt.subplots(figsize=(6, 4))
        im = ax.imshow(m, aspect="auto", cmap="viridis")
        ax.set_xlabel("head")
        ax.set_ylabel("layer")
        ax.set_title(f"{run}: attention entropy (nats)")
        fig.colorbar(im)
        fig.tight_layout()
        fig.savefig(d / "head_entropy_map.png", dpi=120)
        plt.close(fig)
    aw = d / "attention_weights.npz"
    if aw.exists():
        with np.load(aw) as z:
            for key in z.files[:6]:                      # a handful: one image per (prompt, layer), heads side by side
                w = z[key].astype(np.float32)
                n = min(len(w), 8)
                fig, axes = plt.subplots(1, n, figsize=(2 * n, 2.2))
                for h, ax in enumerate(np.atleast_1d(axes)):
                    ax.imshow(w[h], cmap="magma")
                    ax.set_xticks([])
                    ax.set_yticks([])
                    ax.set_title(f"h{h}", fontsize=7)
                fig.suptitle(f"{run}: {key}", fontsize=8)
                fig.savefig(d / f"attention_{key}.png", dpi=110)
                plt.close(fig)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--run", default=None)
    ap.add_argument("--runs", default=None, help="comma-separated runs to overlay (comparison plots go to <output-dir>/_pairs)")
    ap.add_argument("--output-dir", default="analysis")
    ap.add_argument("--input", default=None, help="the directory with one run's extracted files (instead of --run / --output-dir)")
    ap.add_argument("--only", default=None, help="comma-separated series names (or prefixes) to draw; default: all")
    ap.add_argument("--style", default="publication", choices=["publication", "dark", "notebook"], help="matplotlib style of the PNG figures")
    a = ap.parse_args()
    runs = [r.strip() for r in a.runs.split(",")] if a.runs else ([a.run] if a.run else [])
    if a.input:
        d = Path(a.input)
        runs = [d.parent.name if d.name == "activation_geometry" else d.name]
        loaded = {runs[0]: (d, json.loads((d / "geometry.json").read_text()))}
    elif not runs:
        raise SystemExit("give --run, --runs or --input")
    else:
        loaded = {r: load_run(a.output_dir, r) for r in runs}
    all_series = {r: series(geo) for r, (_, geo) in loaded.items()}
    if a.only:
        want = tuple(w.strip() for w in a.only.split(",") if w.strip())
        all_series = {r: {k: v for k, v in s.items() if k.startswith(want)} for r, s in all_series.items()}
    try:
        import matplotlib
        matplotlib.use("Agg")
        import matplotlib.pyplot as plt
        pu.apply_style(plt, dark=a.style == "dark")
    except ImportError:
        plt = None
    for r, (d, _) in loaded.items():
        if plt is None:
            write_csv(d / "series.csv", all_series[r])
            he = d / "head_entropy.npz"
            if he.exists():
                with np.load(he) as z:
                    np.savetxt(d / "head_entropy_map.csv", z["entropy"], delimiter=",", fmt="%.5f")
            n = svg_run(d, r, all_series[r])
            print(f"matplotlib is not installed: {n} SVG figures and series.csv -> {d}")
        else:
            plot_run(plt, d, r, all_series[r])
            print(f"plots -> {d}")
    if len(runs) > 1:
        pd = Path(a.output_dir) / "_pairs"
        pd.mkdir(parents=True, exist_ok=True)
        shared = sorted(set.intersection(*[set(s) for s in all_series.values()]))
        pj = pd / "procrustes.json"
        dist = json.loads(pj.read_text()) if pj.exists() else {}
        if plt is None:
            rows = {f"{k}|{r}": all_series[r][k] for k in shared for r in runs}
            rows.update({f"procrustes|{pair}": v for pair, v in dist.items()})
            write_csv(pd / "comparison.csv", rows)
            for k in shared:
                (pd / f"compare_{k}.svg").write_text(pu.line_chart({r: all_series[r][k] for r in runs}, title=k, xlabel="layer"))
            if dist:
                n = max(len(v) for v in dist.values())
                (pd / "procrustes.svg").write_text(pu.line_chart(dist, title="Procrustes distance between runs", x=list(range(-1, n - 1)),
                                                                 xlabel="layer (-1 = embeddings)"))
            print(f"matplotlib is not installed: {len(shared) + bool(dist)} SVG figures and comparison.csv -> {pd}")
            return
        for k in shared:
            fig, ax = plt.subplots(figsize=(5.5, 3.2))
            for r in runs:
                ax.plot(all_series[r][k], marker="o", ms=3, label=r)
            ax.set_title(k)
            ax.legend(fontsize=7)
            fig.tight_layout()
            fig.savefig(pd / f"compare_{k}.png", dpi=120)
            plt.close(fig)
        if dist:
            fig, ax = plt.subplots(figsize=(5.5, 3.2))
            for pair, v in dist.items():
                ax.plot(range(-1, len(v) - 1), v, marker="o", ms=3, label=pair)
            ax.set_xlabel("layer (-1 = embeddings)")
            ax.set_ylabel("Procrustes distance")
            ax.legend(fontsize=7)
            fig.tight_layout()
            fig.savefig(pd / "procrustes.png", dpi=120)
            plt.close(fig)
        print(f"comparison plots -> {pd}")


if __name__ == "__main__":
    main()
