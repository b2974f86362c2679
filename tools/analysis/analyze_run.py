#!/usr/bin/env python
"""Training-run analyser (tracks 1 and 2): endpoint summary, dynamics (multi-window slopes, inflection
points, rolling statistics, plateaus, jumps), geometric health (per-layer records, landmark profiles,
depth gradient), cross-run comparison with direction-aware deltas, 2x2 factorial analysis and
comparison to a reference, all from ``metrics.jsonl`` / ``geo_metrics.jsonl`` files.

    python tools/analysis/analyze_run.py runs/a/metrics.jsonl --full
    python tools/analysis/analyze_run.py runs/a/metrics.jsonl --dynamics --metrics train/loss,train/grad_norm
    python tools/analysis/analyze_run.py runs/*/metrics.jsonl --compare
    python tools/analysis/analyze_run.py base.jsonl a.jsonl b.jsonl ab.jsonl --factorial "A,B"
    python tools/analysis/analyze_run.py base.jsonl a.jsonl b.jsonl ab.jsonl --factorial "NCA:base,a AttnRes:base,b"
    python tools/analysis/analyze_run.py run.jsonl --reference analysis/base/training.json
    python tools/analysis/analyze_run.py run.jsonl --reference other_run.jsonl

``--factorial`` takes either two factor names (files in the order base, +A, +B, +A+B) or the explicit form
``"A:without,with B:without,with"`` with run names (the fourth file is the run with both factors).
The result is printed as a readable digest and, with ``--output``, written in full as JSON.
Counterpart of the reference's ``scripts/analysis/analyze_run.py``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path
from typing import Any

from _common import write_json

from kotodama_b200.eval import load_metrics
from kotodama_b200.eval import run_analysis as ra


def run_name(path: Path) -> str:
    """Short name of a run from its metrics path: the file stem without the usual suffixes, or the
    directory when the file is just called metrics.jsonl."""
    stem = path.stem
    for suffix in ("_full_metrics", "_metrics", "_full"):
        if stem.endswith(suffix):
            stem = stem[: -len(suffix)]
            break
    if stem in ("metrics", "geo_metrics") and path.parent.name:
        return path.parent.name
    return stem


def parse_factorial(spec: str, names: list[str]) -> tuple[list[str], dict[tuple[int, int], str]]:
    """Factor names and the run of every cell (a, b) of the 2x2 grid."""
    if ":" not in spec:
        factors = [s.strip() for s in spec.split(",")]
        if len(factors) != 2 or len(names) != 4:
            raise SystemExit('--factorial "A,B" needs exactly four metrics files: base, +A, +B, +A+B')
        return factors, {(0, 0): names[0], (1, 0): names[1], (0, 1): names[2], (1, 1): names[3]}
    parts = spec.split()
    if len(parts) != 2:
        raise SystemExit('--factorial: give two factors, e.g. "NCA:base,nca AttnRes:base,ar"')
    factors, pairs = [], []
    for p in parts:
        f, runs = p.split(":", 1)
        without, with_ = [r.strip() for r in runs.split(",")]
        factors.append(f)
        pairs.append((without, with_))
    for without, with_ in pairs:
        for r in (without, with_):
            if r not in names:
                raise SystemExit(f"--factorial: run '{r}' is not among {names}")
    if pairs[0][0] != pairs[1][0]:
        raise SystemExit("--factorial: both factors must name the same run as their 'without' cell")
    both = [n for n in names if n not in (pairs[0][0], pairs[0][1], pairs[1][1])]
    if len(both) != 1:
        raise SystemExit(f"--factorial: cannot tell which run has both factors among {names}")
    return factors, {(0, 0): pairs[0][0], (1, 0): pairs[0][1], (0, 1): pairs[1][1], (1, 1): both[0]}


def fmt(v: Any) -> str:
    if isinstance(v, float):
        return f"{v:.4g}"
    return str(v)


def digest(out: dict[str, Any]) -> str:
    """The result as a few readable lines per section."""
    lines: list[str] = []
    for name, s in out.get("summary", {}).items():
        lines.append(f"[{name}] steps {s.get('max_step')}  loss {fmt(s.get('loss_initial'))} -> {fmt(s.get('loss_final'))} "
                     f"(min {fmt(s.get('loss_min'))} at {s.get('loss_min_step')})"
                     + (f"  rankme {fmt(s.get('rankme_final'))}" if "rankme_final" in s else "")
                     + (f"  {fmt(s.get('avg_tokens_per_sec'))} tok/s" if "avg_tokens_per_sec" in s else ""))
    for name, d in out.get("dynamics", {}).items():
        for key, m in d.items():
            tail = ", ".join(f"{k} {fmt(v)}" for k, v in m.get("slopes", {}).items())
            lines.append(f"[{name}] {key}: slopes {tail}; {len(m.get('plateaus', []))} plateaus, {len(m.get('jumps', []))} jumps, "
                         f"{len(m.get('inflection_points', []))} inflections"
                         + (f", stability {fmt(m['stability_score'])}" if "stability_score" in m else ""))
    for name, g in out.get("geometric_health", {}).items():
        lines.append(f"[{name}] geometry: {len(g.get('layers', {}))} sampled layers, flags {g.get('flags') or 'none'}"
                     + (f", rankme stability {fmt(g['rankme_stability'])}" if "rankme_stability" in g else ""))
    c = out.get("comparison")
    if c:
        lines.append(f"comparison on {c['metric']}: ranking {' < '.join(c['ranking'])}")
        for n, row in c.get("deltas", {}).items():
            verdicts = ", ".join(f"{k} {fmt(v['delta'])} ({v['verdict']})" for k, v in row.items())
            lines.append(f"  {n} vs {c['baseline']}: {verdicts}")
    f = out.get("factorial")
    if f and "interaction" in f:
        a, b = f["factors"]
        lines.append(f"factorial at step {f['step']} on {f['metric']}: {a} {fmt(f['main_effect_a'])}, {b} {fmt(f['main_effect_b'])}, "
                     f"interaction {fmt(f['interaction'])} ({f['classification']}, {fmt(f['relative_interaction'])} of the larger effect)")
    r = out.get("reference")
    if r and "metrics" in r:
        for k, v in r["metrics"].items():
            lines.append(f"vs reference, {k}: {fmt(v['run'])} against {fmt(v['reference'])} (delta {fmt(v['delta'])})")
        if r.get("steps_to_reference_final_loss") is not None:
            lines.append(f"  reaches the reference's final loss at step {r['steps_to_reference_final_loss']}"
                         + (f" ({fmt(r['speedup_vs_reference'])}x fewer steps)" if "speedup_vs_reference" in r else ""))
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("metrics", nargs="+", help="JSONL metrics file(s)")
    ap.add_argument("--name", default=None, help="run name (single file) instead of the one taken from the path")
    ap.add_argument("--summary", action="store_true")
    ap.add_argument("--dynamics", action="store_true")
    ap.add_argument("--geometry", "--health", dest="geometry", action="store_true")
    ap.add_argument("--full", action="store_true", help="summary + dynamics + geometry")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--factorial", default=None, help='"A,B" (files: base, +A, +B, +A+B) or "A:without,with B:without,with"')
    ap.add_argument("--reference", default=None, help="JSON written by this tool (its summary is used), or another metrics file")
    ap.add_argument("--metric", default="train/loss", help="metric of --compare / --factorial")
    ap.add_argument("--metrics", dest="metric_list", default=None, help="comma-separated metrics for --dynamics (default: loss, RankMe)")
    ap.add_argument("--output", "-o", default=None, help="write the full result as JSON here")
    ap.add_argument("--quiet", action="store_true", help="no digest on stdout")
    a = ap.parse_args()
    paths = [Path(p) for p in a.metrics]
    names = [a.name] if a.name and len(paths) == 1 else [run_name(p) for p in paths]
    if len(set(names)) != len(names):                    # same stem in different folders
        names = [f"{p.parent.name}/{n}" for p, n in zip(paths, names)]
    runs = {n: load_metrics(p) for n, p in zip(names, paths)}
    keys = [k.strip() for k in a.metric_list.split(",")] if a.metric_list else None
    out: dict[str, Any] = {}
    first = next(iter(runs.values()))
    if a.summary or a.full or not (a.dynamics or a.geometry or a.compare or a.factorial or a.reference):
        out["summary"] = {n: ra.endpoint_summary(d) for n, d in runs.items()}
    if a.dynamics or a.full:
        out["dynamics"] = {n: ra.training_dynamics(d, keys) for n, d in runs.items()}
    if a.geometry or a.full:
        out["geometric_health"] = {n: ra.geometric_health(d) for n, d in runs.items()}
    if a.compare and len(runs) > 1:
        out["comparison"] = ra.compare_runs(runs, metric=a.metric)
    if a.factorial:
        factors, cells = parse_factorial(a.factorial, names)
        out["factorial"] = {"factors": factors, "cells": {f"{k[0]}{k[1]}": v for k, v in cells.items()},
                            **ra.factorial_analysis({k: runs[v] for k, v in cells.items()}, metric=a.metric,
                                                    extra_metrics=[k for k in (keys or ["geo/rankme_last"]) if k != a.metric])}
    if a.reference:
        ref = Path(a.reference)
        if ref.suffix == ".json":
            stored = json.loads(ref.read_text())
            if "summary" in stored and isinstance(stored["summary"], dict):      # a result of this tool: first run's summary
                stored = next(iter(stored["summary"].values()))
            mine = ra.endpoint_summary(first)
            out["reference"] = {"endpoints": {k: {"run": mine.get(k), "reference": stored.get(k),
                                                  "delta": (mine[k] - stored[k]) if isinstance(mine.get(k), (int, float)) and isinstance(stored.get(k), (int, float)) else None}
                                              for k in sorted(set(mine) | set(stored))
                                              if isinstance(mine.get(k), (int, float)) or isinstance(stored.get(k), (int, float))}}
        else:
            out["reference"] = ra.reference_comparison(first, load_metrics(ref), keys)
    if a.output:
        write_json(Path(a.output), out)
    if not a.quiet:
        text = digest(out)
        print(text if text else json.dumps(out, indent=1, default=str))
        if a.output:
            print(f"-> {a.output}")


if __name__ == "__main__":
    main()
