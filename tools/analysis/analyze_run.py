#!/usr/bin/env python
"""Training-run analyser (tracks 1 and 2): endpoint summary, dynamics (slopes, plateaus, jumps),
geometric health, cross-run comparison, 2x2 factorial analysis and comparison to a stored
reference summary, all from ``metrics.jsonl`` / ``geo_metrics.jsonl`` files.

    python tools/analysis/analyze_run.py runs/a/metrics.jsonl --full
    python tools/analysis/analyze_run.py runs/*/metrics.jsonl --compare
    python tools/analysis/analyze_run.py base.jsonl a.jsonl b.jsonl ab.jsonl --factorial "A,B"
    python tools/analysis/analyze_run.py run.jsonl --reference analysis/base/training_summary.json

Counterpart of the reference's ``scripts/analysis/analyze_run.py``.
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

from _common import write_json

from kotodama_b200.eval import load_metrics
from kotodama_b200.eval import run_analysis as ra


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("metrics", nargs="+")
    ap.add_argument("--summary", action="store_true")
    ap.add_argument("--dynamics", action="store_true")
    ap.add_argument("--geometry", action="store_true")
    ap.add_argument("--full", action="store_true")
    ap.add_argument("--compare", action="store_true")
    ap.add_argument("--factorial", default=None, help='"A,B": files are given in the order base, +A, +B, +A+B')
    ap.add_argument("--reference", default=None, help="JSON with a stored endpoint summary, or another metrics file")
    ap.add_argument("--metric", default="train/loss")
    ap.add_argument("--output", default=None, help="write the result as JSON here (default: print)")
    a = ap.parse_args()
    runs = {Path(p).parent.name + "/" + Path(p).stem if Path(p).parent.name else Path(p).stem: load_metrics(p)
            for p in a.metrics}
    out: dict = {}
    first = next(iter(runs.values()))
    if a.summary or a.full or not (a.dynamics or a.geometry or a.compare or a.factorial or a.reference):
        out["summary"] = {n: ra.endpoint_summary(d) for n, d in runs.items()}
    if a.dynamics or a.full:
        out["dynamics"] = {n: ra.training_dynamics(d) for n, d in runs.items()}
    if a.geometry or a.full:
        out["geometric_health"] = {n: ra.geometric_health(d) for n, d in runs.items()}
    if a.compare and len(runs) > 1:
        out["comparison"] = ra.compare_runs(runs, metric=a.metric)
    if a.factorial:
        if len(runs) != 4:
            raise SystemExit("--factorial needs exactly four metrics files: base, +A, +B, +A+B")
        names = [s.strip() for s in a.factorial.split(",")]
        vals = list(runs.values())
        cells = {(0, 0): vals[0], (1, 0): vals[1], (0, 1): vals[2], (1, 1): vals[3]}
        out["factorial"] = {"factors": names, **ra.factorial_analysis(cells, metric=a.metric)}
    if a.reference:
        ref = Path(a.reference)
        if ref.suffix == ".json":
            stored = json.loads(ref.read_text())
            mine = ra.endpoint_summary(first)
            out["reference"] = {k: {"run": mine.get(k), "reference": stored.get(k)} for k in sorted(set(mine) | set(stored))
                                if isinstance(mine.get(k), (int, float)) or isinstance(stored.get(k), (int, float))}
        else:
            out["reference"] = ra.reference_comparison(first, load_metrics(ref))
    if a.output:
        write_json(Path(a.output), out)
    else:
        print(json.dumps(out, indent=1, default=str))


if __name__ == "__main__":
    main()
