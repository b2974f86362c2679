#!/usr/bin/env python
"""Self-contained HTML report of one run from the outputs of the analysis tracks that exist under
``<output-dir>/<run>/``: training summary / dynamics / geometric health (``training.json`` from
``analyze_run.py --full --output``), generations + perplexity, text quality, activation geometry,
concept geometry.  With ``--metrics`` (or a ``metrics.jsonl`` / ``geo_metrics.jsonl`` next to the data) the
report also draws the curves themselves: loss and learning rates, gradient norm, throughput, RankMe and
stable ranks over training, the per-layer depth profile at the last step, AttnRes routing weights.  Charts
are inline SVG (line charts with axes and legend, bar profiles, a radar of text-quality scores), images
found next to the data are embedded as base64; the page opens with cards of the run's headline numbers.

    python tools/analysis/generate_report.py my-run [--output-dir analysis] [--metrics runs/my-run/metrics.jsonl] \
        [--theme light] [-o report.html]

Counterpart of the reference's ``scripts/analysis/generate_report.py``.
"""
from __future__ import annotations

import argparse
import base64
import html
import json
import math
import os
import sys
from datetime import datetime
from pathlib import Path
from typing import Any, Optional, Sequence

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", ".."))

THEMES = {"dark": ("#14161a", "#e6e6e6", "#7fb4ff", "#23262d"), "light": ("#ffffff", "#1b1b1b", "#1f5fbf", "#f1f3f6")}


def load(p: Path) -> Optional[Any]:
    return json.loads(p.read_text()) if p.exists() else None


def spark(values: list[float], colour: str, w: int = 360, h: int = 90) -> str:
    vals = [float(v) for v in values if v is not None]
    if len(vals) < 2:
        return ""
    lo, hi = min(vals), max(vals)
    span = (hi - lo) or 1.0
    pts = " ".join(f"{i * (w - 10) / (len(vals) - 1) + 5:.1f},{h - 8 - (v - lo) / span * (h - 16):.1f}" for i, v in enumerate(vals))
    return (f'<svg width="{w}" height="{h}" viewBox="0 0 {w} {h}"><polyline fill="none" stroke="{colour}" stroke-width="1.6" '
            f'points="{pts}"/><text x="5" y="10" font-size="9" fill="{colour}">{hi:.4g}</text>'
            f'<text x="5" y="{h - 1}" font-size="9" fill="{colour}">{lo:.4g}</text></svg>')


PALETTE = ["#4e9af1", "#f1a14e", "#6fcf97", "#eb5757", "#bb6bd9", "#56ccf2", "#f2c94c", "#9b9b9b"]


def _ticks(lo: float, hi: float, n: int = 4) -> list[float]:
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 5, 10) if m * mag >= raw), default=raw)
    first = math.ceil(lo / step) * step
    out, v = [], first
    while v <= hi + 1e-12:
        out.append(v)
        v += step
    return out or [lo, hi]


def line_chart(series: dict[str, Sequence[tuple[float, float]]], fg: str, title: str = "", log_y: bool = False,
               w: int = 560, h: int = 230) -> str:
    """Several (x, y) series on shared axes: grid, ticks, legend.  ``log_y`` plots log10(y)."""
    series = {k: [(float(x), float(y)) for x, y in v if y is not None and (not log_y or y > 0)] for k, v in series.items()}
    series = {k: v for k, v in series.items() if len(v) >= 2}
    if not series:
        return ""
    tf = (lambda y: math.log10(y)) if log_y else (lambda y: y)
    xs = [x for v in series.values() for x, _ in v]
    ys = [tf(y) for v in series.values() for _, y in v]
    x0, x1, y0, y1 = min(xs), max(xs), min(ys), max(ys)
    if y1 == y0:
        y1 = y0 + 1
    pad_l, pad_r, pad_t, pad_b = 52, 12, 22, 26
    px = lambda x: pad_l + (x - x0) / ((x1 - x0) or 1) * (w - pad_l - pad_r)
    py = lambda y: h - pad_b - (y - y0) / (y1 - y0) * (h - pad_t - pad_b)
    out = [f'<svg width="{w}" height="{h}" viewBox="0 0 {w} {h}" font-size="10" fill="{fg}">']
    if title:
        out.append(f'<text x="{pad_l}" y="13" font-size="12">{html.escape(title)}</text>')
    for t in _ticks(y0, y1):
        lab = f"{10 ** t:.3g}" if log_y else f"{t:.4g}"
        out.append(f'<line x1="{pad_l}" x2="{w - pad_r}" y1="{py(t):.1f}" y2="{py(t):.1f}" stroke="{fg}" stroke-opacity=".15"/>'
                   f'<text x="{pad_l - 5}" y="{py(t) + 3:.1f}" text-anchor="end">{lab}</text>')
    for t in _ticks(x0, x1, 5):
        out.append(f'<text x="{px(t):.1f}" y="{h - 8}" text-anchor="middle">{t:.6g}</text>')
    out.append(f'<rect x="{pad_l}" y="{pad_t}" width="{w - pad_l - pad_r}" height="{h - pad_t - pad_b}" fill="none" '
               f'stroke="{fg}" stroke-opacity=".4"/>')
    for i, (name, pts) in enumerate(series.items()):
        step = max(1, len(pts) // 600)                    # thin very long curves
        pl = " ".join(f"{px(x):.1f},{py(tf(y)):.1f}" for x, y in pts[::step])
        col = PALETTE[i % len(PALETTE)]
        out.append(f'<polyline fill="none" stroke="{col}" stroke-width="1.5" points="{pl}"/>')
        out.append(f'<rect x="{w - pad_r - 150}" y="{pad_t + 6 + 13 * i}" width="9" height="9" fill="{col}"/>'
                   f'<text x="{w - pad_r - 137}" y="{pad_t + 14 + 13 * i}">{html.escape(name[:26])}</text>')
    out.append("</svg>")
    return "".join(out)


def bar_profile(labels: Sequence[str], values: Sequence[float], fg: str, colour: str, title: str = "", w: int = 560, h: int = 170) -> str:
    """One bar per label (a per-layer depth profile)."""
    vals = [float(v) for v in values]
    if not vals:
        return ""
    hi, lo = max(vals + [0.0]), min(vals + [0.0])
    span = (hi - lo) or 1.0
    pad_l, pad_b, pad_t = 46, 24, 20
    bw = (w - pad_l - 8) / len(vals)
    zero = h - pad_b - (0 - lo) / span * (h - pad_t - pad_b)
    out = [f'<svg width="{w}" height="{h}" viewBox="0 0 {w} {h}" font-size="10" fill="{fg}">']
    if title:
        out.append(f'<text x="{pad_l}" y="12" font-size="12">{html.escape(title)}</text>')
    out.append(f'<text x="{pad_l - 4}" y="{pad_t + 8}" text-anchor="end">{hi:.3g}</text>'
               f'<text x="{pad_l - 4}" y="{h - pad_b}" text-anchor="end">{lo:.3g}</text>')
    for i, v in enumerate(vals):
        y = h - pad_b - (v - lo) / span * (h - pad_t - pad_b)
        out.append(f'<rect x="{pad_l + i * bw + 1:.1f}" y="{min(y, zero):.1f}" width="{max(bw - 2, 1):.1f}" height="{abs(zero - y):.1f}" '
                   f'fill="{colour}"/>')
        if len(vals) <= 32 or i % 4 == 0:
            out.append(f'<text x="{pad_l + (i + .5) * bw:.1f}" y="{h - 8}" text-anchor="middle">{html.escape(str(labels[i]))}</text>')
    out.append("</svg>")
    return "".join(out)


def radar(labels: Sequence[str], values: Sequence[float], fg: str, colour: str, size: int = 300) -> str:
    """Scores in [0, 1] on spokes."""
    n = len(labels)
    if n < 3:
        return ""
    c, r = size / 2, size / 2 - 46
    pt = lambda i, v: (c + r * v * math.sin(2 * math.pi * i / n), c - r * v * math.cos(2 * math.pi * i / n))
    out = [f'<svg width="{size + 120}" height="{size}" viewBox="-60 0 {size + 120} {size}" font-size="10" fill="{fg}">']
    for ring in (0.25, 0.5, 0.75, 1.0):
        out.append('<polygon fill="none" stroke="%s" stroke-opacity=".2" points="%s"/>'
                   % (fg, " ".join("%.1f,%.1f" % pt(i, ring) for i in range(n))))
    for i, lab in enumerate(labels):
        x, y = pt(i, 1.0)
        lx, ly = pt(i, 1.16)
        out.append(f'<line x1="{c}" y1="{c}" x2="{x:.1f}" y2="{y:.1f}" stroke="{fg}" stroke-opacity=".2"/>'
                   f'<text x="{lx:.1f}" y="{ly:.1f}" text-anchor="middle">{html.escape(lab)}</text>')
    out.append('<polygon fill="%s" fill-opacity=".3" stroke="%s" stroke-width="1.5" points="%s"/>'
               % (colour, colour, " ".join("%.1f,%.1f" % pt(i, max(0.0, min(1.0, v))) for i, v in enumerate(values))))
    out.append("</svg>")
    return "".join(out)


def cards(items: Sequence[tuple[str, str, str]], panel: str, ac: str) -> str:
    return '<div class="cards">' + "".join(
        f'<div class="card"><div class="v" style="color:{ac}">{html.escape(v)}</div><div class="l">{html.escape(l)}</div>'
        f'<div class="s">{html.escape(sub)}</div></div>' for l, v, sub in items) + "</div>"


def series_of(data: dict[int, dict[str, float]], key: str) -> list[tuple[int, float]]:
    return [(s, rec[key]) for s, rec in sorted(data.items()) if isinstance(rec.get(key), (int, float))]


def training_charts(data: dict[int, dict[str, float]], fg: str, ac: str) -> tuple[str, list[tuple[str, str, str]]]:
    """Curves and headline cards from a metrics file (the keys the training driver logs)."""
    body, hero = "", []
    loss = {k.split("/", 1)[1]: series_of(data, k) for k in ("train/loss", "val/loss", "train/z_loss") if series_of(data, k)}
    body += line_chart(loss, fg, "loss", log_y=False)
    lrs = {k.split("/", 1)[1]: series_of(data, k) for k in ("train/lr_muon", "train/lr_adamw", "train/lr") if series_of(data, k)}
    body += line_chart(lrs, fg, "learning rates")
    gn = {k.split("/", 1)[1]: series_of(data, k) for k in ("train/grad_norm", "train/grad_norm_preclip") if series_of(data, k)}
    body += line_chart(gn, fg, "gradient norm", log_y=True)
    tps = series_of(data, "perf/tokens_per_sec")
    body += line_chart({"tokens/s": tps}, fg, "throughput")
    rk = {k.split("/", 1)[1]: series_of(data, k) for k in ("geo/rankme_last", "geo/ww_alpha_mean", "geo/ww_alpha_healthy_frac")
          if series_of(data, k)}
    body += line_chart(rk, fg, "representation health")
    # depth profiles at the last step that carries them: per-layer gradient norms, intrinsic dimension, routing weights
    def latest(prefix: str) -> list[tuple[str, float]]:
        order = lambda kv: int("".join(ch for ch in kv[0] if ch.isdigit()) or 0)
        for _, rec in sorted(data.items(), reverse=True):
            items = sorted(((k[len(prefix):], v) for k, v in rec.items() if k.startswith(prefix)), key=order)
            if items:
                return items
        return []
    for prefix, title in (("grad_norm/layer_", "gradient norm per layer (last step)"), ("geo/twonn_id/layer_", "intrinsic dimension per layer"),
                          ("attnres/final_alpha/", "AttnRes output routing weight per source")):
        items = latest(prefix)
        if items:
            body += bar_profile([k for k, _ in items], [v for _, v in items], fg, ac, title)
    sr = {}
    for _, rec in sorted(data.items(), reverse=True):
        sr = {k: v for k, v in rec.items() if k.startswith("geo/layer_") and "/stable_rank_" in k}
        if sr:
            break
    by_proj: dict[str, list[tuple[int, float]]] = {}
    for k, v in sr.items():
        layer = int(k.split("/")[1].split("_")[1])
        by_proj.setdefault(k.split("stable_rank_")[1], []).append((layer, v))
    body += line_chart({p: sorted(v) for p, v in by_proj.items()}, fg, "stable rank per layer and projection")
    if loss.get("loss"):
        hero.append(("final train loss", f"{loss['loss'][-1][1]:.4f}", f"min {min(v for _, v in loss['loss']):.4f}"))
    if series_of(data, "val/loss"):
        v = series_of(data, "val/loss")
        hero.append(("validation loss", f"{v[-1][1]:.4f}", f"best {min(x for _, x in v):.4f}"))
    if tps:
        stable = tps[2:] or tps
        hero.append(("throughput", f"{sum(v for _, v in stable) / len(stable) / 1e3:.1f} K tok/s", "mean after warm-up"))
    tok = series_of(data, "data/tokens_consumed_B")
    if tok:
        hero.append(("tokens", f"{tok[-1][1]:.3g} B", f"{max(data)} steps"))
    elif data:
        hero.append(("steps", str(max(data)), ""))
    return body, hero


def quality_radar(tq: dict[str, Any], fg: str, ac: str) -> str:
    """Six scores in [0, 1] from the text-quality metrics (higher = better)."""
    o = tq.get("overall", {})
    g = lambda fam, k, d=0.0: float(o.get(fam, {}).get(k, d))
    clamp = lambda v: max(0.0, min(1.0, v))
    scores = {
        "diversity": clamp(g("lexical", "ttr_100", g("lexical", "mattr_100"))),
        "non-repetition": clamp(g("repetition", "unique_3gram_ratio", g("repetition", "distinct_3"))),
        "coherence": clamp(g("coherence", "topic_similarity_mean", g("coherence", "adjacent_jaccard")) * 2.5),
        "structure": clamp(g("structural", "clause_depth_mean", 1.0) / 3.0),
        "specificity": clamp(g("creativity", "specificity_score") / 10.0),
        "completion": clamp(g("creativity", "ends_terminated", g("commitment", "ends_terminated"))),
        "no loops": clamp(1.0 - float(o.get("loop_rate", 0.0))),
    }
    return radar(list(scores), list(scores.values()), fg, ac)


def table(rows: list[tuple[str, Any]]) -> str:
    def fmt(v: Any) -> str:
        if isinstance(v, float):
            return f"{v:.4g}"
        return html.escape(str(v))
    return "<table>" + "".join(f"<tr><th>{html.escape(str(k))}</th><td>{fmt(v)}</td></tr>" for k, v in rows) + "</table>"


def flat(d: Any, prefix: str = "") -> list[tuple[str, Any]]:
    out = []
    if isinstance(d, dict):
        for k, v in d.items():
            out += flat(v, f"{prefix}{k}." if isinstance(v, dict) else f"{prefix}{k}")
    else:
        out.append((prefix.rstrip("."), d))
    return [(k, v) for k, v in out if not isinstance(v, (list, dict))]


def images(d: Path) -> str:
    """The figures the visualisers left in ``d``: PNG (matplotlib) as data URIs, SVG (built-in plotting layer) inline."""
    out = []
    for p in sorted(d.glob("*.png")):
        out.append(f'<figure><img src="data:image/png;base64,{base64.b64encode(p.read_bytes()).decode()}"/>'
                   f"<figcaption>{html.escape(p.stem)}</figcaption></figure>")
    for p in sorted(d.glob("*.svg")):
        if not (d / (p.stem + ".png")).exists():
            out.append(f"<figure>{p.read_text()}<figcaption>{html.escape(p.stem)}</figcaption></figure>")
    return "".join(out)


def build(run: str, rd: Path, theme: str, metrics: Optional[Path] = None) -> str:
    bg, fg, ac, panel = THEMES[theme]
    sec = []
    hero: list[tuple[str, str, str]] = []
    mfiles = [p for p in ([metrics] if metrics else [rd / "metrics.jsonl"]) if p and p.exists()]
    if mfiles:
        from kotodama_b200.eval import load_metrics
        data = load_metrics(mfiles[0])
        geo_file = mfiles[0].with_name("geo_metrics.jsonl")
        if geo_file.exists():
            for st, rec in load_metrics(geo_file).items():
                data.setdefault(st, {}).update(rec)
        body, hero = training_charts(data, fg, ac)
        if body:
            sec.append(("Training curves", body))
    tr = load(rd / "training.json")
    if tr:
        for part in ("summary", "dynamics", "geometric_health"):
            if part in tr:
                body = "".join(f"<h4>{html.escape(n)}</h4>" + table(flat(v)[:40]) for n, v in tr[part].items())
                sec.append((f"Training: {part.replace('_', ' ')}", body))
    gen = load(rd / "generations.json")
    if gen:
        body = table(flat(gen.get("config", {})) + flat({"perplexity": gen.get("perplexity", {})}))
        ppl = gen.get("perplexity", {})
        if isinstance(ppl, dict) and ppl:
            k0 = next(iter(ppl))
            v0 = ppl[k0]["perplexity"] if isinstance(ppl[k0], dict) and "perplexity" in ppl[k0] else ppl[k0]
            if isinstance(v0, (int, float)):
                hero.append(("perplexity", f"{v0:.2f}", str(k0)))
        for g in gen["generations"][:12]:
            body += f"<h4>{html.escape(g['prompt'])}</h4>" + "".join(f"<pre>{html.escape(s[:1500])}</pre>" for s in g["samples"][:2])
        sec.append(("Generations", body))
    tq = load(rd / "text_quality.json")
    if tq:
        sec.append(("Text quality", quality_radar(tq, fg, ac) + table(flat(tq.get("overall", {})))))
        hero.append(("samples scored", str(tq.get("overall", {}).get("n", 0)),
                     f"loop rate {float(tq.get('overall', {}).get('loop_rate', 0.0)):.2f}"))
    geo = load(rd / "activation_geometry" / "geometry.json")
    if geo:
        body = ""
        if "eigenspectra" in geo:
            body += "<h4>RankMe per layer</h4>" + spark([e["rankme"] for e in geo["eigenspectra"]], ac)
            body += "<h4>Participation ratio per layer</h4>" + spark([e["participation_ratio"] for e in geo["eigenspectra"]], ac)
        if "trajectories" in geo:
            body += "<h4>Mean state norm per layer</h4>" + spark(geo["trajectories"]["mean_norm_per_layer"], ac)
        for l, a in geo.get("attention", {}).items():
            body += f"<h4>Head entropy, layer {l}</h4>" + spark(a["head_entropy"], ac)
        if "head_entropy" in geo:
            body += "<h4>Mean head entropy per layer (all layers)</h4>" + spark(geo["head_entropy"]["mean_per_layer"], ac)
        if "attention_outputs" in geo:
            body += "<h4>Attention branch norm / state norm per layer</h4>" + spark(geo["attention_outputs"]["branch_to_state_norm_ratio"], ac)
        twonn = geo.get("topo_clouds", {}).get("twonn_dimension")
        if twonn:
            body += "<h4>TwoNN intrinsic dimension of the token clouds</h4>" + table([(f"layer {k}", float(v)) for k, v in twonn.items()])
        for wtype, m in geo.get("effective_rank", {}).items():
            if isinstance(m, dict) and "participation_ratio" in m:
                body += f"<h4>Effective rank of {html.escape(wtype)} per layer</h4>" + spark(m["participation_ratio"], ac)
        if "trajectories" in geo and "straightness" in geo["trajectories"]:
            hero.append(("trajectory straightness", f"{geo['trajectories']['straightness']:.2f}", "net / path length through depth"))
        body += images(rd / "activation_geometry")
        sec.append(("Activation geometry", body))
    cg = load(rd / "concept_geometry" / "analysis.json")
    if cg:
        body = ""
        for name, s in cg["sets"].items():
            body += f"<h4>{html.escape(name)} ({s['kind']})</h4>"
            if "best_layer" in s:
                body += table(flat(s["best_layer"]))
            key = s["kind"] if s["kind"] in ("cyclic", "ordinal", "geographic") else None
            if key and s["per_layer"] and key in s["per_layer"][0]:
                body += spark([r[key]["r"] for r in s["per_layer"]], ac)
            if s["kind"] == "paired" and s["per_layer"] and "paired" in s["per_layer"][0]:
                body += spark([r["paired"]["completion_accuracy"] for r in s["per_layer"]], ac)
            if s.get("first_significant_layer") is not None:
                body += f"<p>structure significant (p &lt; 0.05) from layer {s['first_significant_layer']} on, in {s['significant_layers']} layers</p>"
        if cg.get("summary"):
            found = [n for n, v in cg["summary"].items() if v.get("p", 1.0) < 0.05]
            hero.append(("concept sets with structure", f"{len(found)} / {len(cg['summary'])}", "Mantel p < 0.05 at the best layer"))
        body += images(rd / "concept_geometry")
        sec.append(("Concept geometry", body))
    if not sec:
        sec.append(("No data", f"<p>No analysis outputs found under {html.escape(str(rd))}.</p>"))
    nav = "".join(f'<a href="#s{i}">{html.escape(t)}</a>' for i, (t, _) in enumerate(sec))
    body = (cards(hero, panel, ac) if hero else "") + "".join(
        f'<section id="s{i}"><h2>{html.escape(t)}</h2>{b}</section>' for i, (t, b) in enumerate(sec))
    css = (f"body{{background:{bg};color:{fg};font:14px/1.45 system-ui,sans-serif;margin:0 auto;max-width:1000px;padding:24px}}"
           f"a{{color:{ac};margin-right:14px}}section{{background:{panel};border-radius:8px;padding:12px 18px;margin:16px 0}}"
           f"table{{border-collapse:collapse}}th{{text-align:left;padding:2px 14px 2px 0;font-weight:500;opacity:.8}}"
           f"pre{{white-space:pre-wrap;background:{bg};padding:8px;border-radius:6px}}figure{{display:inline-block;margin:6px}}"
           "img{max-width:440px}figcaption{font-size:11px;opacity:.7}svg{margin:4px 8px 4px 0}"
           f".cards{{display:flex;flex-wrap:wrap;gap:12px;margin:14px 0}}.card{{background:{panel};border-radius:8px;padding:10px 16px;min-width:130px}}"
           ".card .v{font-size:22px;font-weight:600}.card .l{font-size:12px;opacity:.85}.card .s{font-size:11px;opacity:.6}")
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(run)} analysis</title><style>{css}</style></head>"
            f"<body><h1>{html.escape(run)}</h1><p>generated {datetime.now():%Y-%m-%d %H:%M}</p><nav>{nav}</nav>{body}</body></html>")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("run")
    ap.add_argument("--output-dir", "--analysis-dir", dest="output_dir", default="analysis")
    ap.add_argument("--metrics", default=None, help="metrics.jsonl of the run (default: <output-dir>/<run>/metrics.jsonl if present)")
    ap.add_argument("--theme", default="dark", choices=list(THEMES))
    ap.add_argument("-o", "--output", default=None)
    a = ap.parse_args()
    rd = Path(a.output_dir) / a.run
    dst = Path(a.output) if a.output else rd / "report.html"
    dst.parent.mkdir(parents=True, exist_ok=True)
    dst.write_text(build(a.run, rd, a.theme, Path(a.metrics) if a.metrics else None))
    print(f"report -> {dst}")


if __name__ == "__main__":
    main()
