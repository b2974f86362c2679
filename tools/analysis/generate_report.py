#!/usr/bin/env python
"""Self-contained HTML report of one run from the outputs of the analysis tracks that exist under
``<output-dir>/<run>/``: training summary / dynamics / geometric health (``training.json`` from
``analyze_run.py --full --output``), generations + perplexity, text quality, activation geometry,
concept geometry.  Charts are inline SVG, images found next to the data are embedded as base64.

    python tools/analysis/generate_report.py my-run [--output-dir analysis] [--theme light] [-o report.html]

Counterpart of the reference's ``scripts/analysis/generate_report.py``.
"""
from __future__ import annotations

import argparse
import base64
import html
import json
from datetime import datetime
from pathlib import Path
from typing import Any, Optional

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
    out = []
    for p in sorted(d.glob("*.png")):
        out.append(f'<figure><img src="data:image/png;base64,{base64.b64encode(p.read_bytes()).decode()}"/>'
                   f"<figcaption>{html.escape(p.stem)}</figcaption></figure>")
    return "".join(out)


def build(run: str, rd: Path, theme: str) -> str:
    bg, fg, ac, panel = THEMES[theme]
    sec = []
    tr = load(rd / "training.json")
    if tr:
        for part in ("summary", "dynamics", "geometric_health"):
            if part in tr:
                body = "".join(f"<h4>{html.escape(n)}</h4>" + table(flat(v)[:40]) for n, v in tr[part].items())
                sec.append((f"Training: {part.replace('_', ' ')}", body))
    gen = load(rd / "generations.json")
    if gen:
        body = table(flat(gen.get("config", {})) + flat({"perplexity": gen.get("perplexity", {})}))
        for g in gen["generations"][:12]:
            body += f"<h4>{html.escape(g['prompt'])}</h4>" + "".join(f"<pre>{html.escape(s[:1500])}</pre>" for s in g["samples"][:2])
        sec.append(("Generations", body))
    tq = load(rd / "text_quality.json")
    if tq:
        sec.append(("Text quality", table(flat(tq.get("overall", {})))))
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
        body += images(rd / "activation_geometry")
        sec.append(("Activation geometry", body))
    cg = load(rd / "concept_geometry" / "analysis.json")
    if cg:
        body = ""
        for name, s in cg["sets"].items():
            body += f"<h4>{html.escape(name)} ({s['kind']})</h4>"
            if "best_layer" in s:
                body += table(flat(s["best_layer"]))
            key = s["kind"] if s["kind"] in ("cyclic", "ordinal") else None
            if key and s["per_layer"] and key in s["per_layer"][0]:
                body += spark([r[key]["r"] for r in s["per_layer"]], ac)
        body += images(rd / "concept_geometry")
        sec.append(("Concept geometry", body))
    if not sec:
        sec.append(("No data", f"<p>No analysis outputs found under {html.escape(str(rd))}.</p>"))
    nav = "".join(f'<a href="#s{i}">{html.escape(t)}</a>' for i, (t, _) in enumerate(sec))
    body = "".join(f'<section id="s{i}"><h2>{html.escape(t)}</h2>{b}</section>' for i, (t, b) in enumerate(sec))
    css = (f"body{{background:{bg};color:{fg};font:14px/1.45 system-ui,sans-serif;margin:0 auto;max-width:1000px;padding:24px}}"
           f"a{{color:{ac};margin-right:14px}}section{{background:{panel};border-radius:8px;padding:12px 18px;margin:16px 0}}"
           f"table{{border-collapse:collapse}}th{{text-align:left;padding:2px 14px 2px 0;font-weight:500;opacity:.8}}"
           f"pre{{white-space:pre-wrap;background:{bg};padding:8px;border-radius:6px}}figure{{display:inline-block;margin:6px}}"
           "img{max-width:440px}figcaption{font-size:11px;opacity:.7}")
    return (f"<!doctype html><html><head><meta charset='utf-8'><title>{html.escape(run)} analysis</title><style>{css}</style></head>"
            f"<body><h1>{html.escape(run)}</h1><p>generated {datetime.now():%Y-%m-%d %H:%M}</p><nav>{nav}</nav>{body}</body></html>")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("run")
    ap.add_argument("--output-dir", default="analysis")
    ap.add_argument("--theme", default="dark", choices=list(THEMES))
    ap.add_argument("-o", "--output", default=None)
    a = ap.parse_args()
    rd = Path(a.output_dir) / a.run
    dst = Path(a.output) if a.output else rd / "report.html"
    dst.parent.mkdir(parents=True, exist_ok=True)
    dst.write_text(build(a.run, rd, a.theme))
    print(f"report -> {dst}")


if __name__ == "__main__":
    main()
