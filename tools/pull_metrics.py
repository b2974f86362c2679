#!/usr/bin/env python
"""Print an endpoint summary (and optionally training dynamics) of one or more runs from their
``metrics.jsonl`` files:  python tools/pull_metrics.py checkpoints/run-a checkpoints/run-b [--dynamics]"""
import json
import os
import sys

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.eval import load_metrics, run_analysis  # noqa: E402


def main() -> None:
    dyn = "--dynamics" in sys.argv
    runs = {}
    for d in [a for a in sys.argv[1:] if not a.startswith("--")]:
        p = d if d.endswith(".jsonl") else os.path.join(d, "metrics.jsonl")
        runs[os.path.basename(os.path.dirname(os.path.abspath(p)))] = load_metrics(p)
    for name, data in runs.items():
        print(json.dumps({"run": name, **run_analysis.endpoint_summary(data)}))
        if dyn:
            print(json.dumps({"run": name, "dynamics": run_analysis.training_dynamics(data)}))
    if len(runs) > 1:
        print(json.dumps({"ranking": run_analysis.compare_runs(runs)["ranking"]}))


if __name__ == "__main__":
    main()
