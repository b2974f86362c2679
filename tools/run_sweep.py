#!/usr/bin/env python
"""Run a sweep - a named set of training arms that differ in a few flags - on the GPUs of this node, one arm after
the other, and compare the arms when they are done.

    python tools/run_sweep.py configs/sweeps/proxy.yaml --data_path data/train.bin
    python tools/run_sweep.py configs/sweeps/decay.yaml --only sqrt-90,cosine-90 --gpus 4
    python tools/run_sweep.py configs/sweeps/proxy.yaml --dry-run                    # the commands only
    python tools/run_sweep.py my_sweep.yaml --out outputs/my-sweep -- --fp8          # flags after -- go to every arm

A sweep file names a base configuration (``base``), flags shared by all arms (``common``) and the arms themselves
(``experiments``: name -> flags; ``true`` for a switch).  Every arm gets its own directory ``<out>/<arm>/`` with its
checkpoints, ``metrics.jsonl`` (every arm runs with ``--wandb``, which also writes the JSONL files and stays offline
without an API key) and ``train.log``; an arm whose directory already holds ``DONE`` is skipped, so an
interrupted sweep continues where it stopped (the trainer itself resumes an arm from its newest checkpoint).  At the end
the arms are compared on their metrics (endpoint summaries, ranking by final loss, deltas against the first arm) and
the result is written to ``<out>/sweep_summary.json``.

The reference drives its sweeps with shell loops and cluster submitters (``scripts/legacy/run_*_sweep.sh``,
``submit_*_sweep.py``); this is the same job for one node, without any scheduler or credentials.
"""
from __future__ import annotations

import argparse
import datetime
import json
import sys
from pathlib import Path
from typing import Any

import yaml

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT))
sys.path.insert(0, str(ROOT / "tools"))
from benchmark_matrix import gpu_count, run_one, trainer_command  # noqa: E402

from kotodama_b200.eval import load_metrics, run_analysis  # noqa: E402


def flags_of(settings: dict[str, Any]) -> list[str]:
    """``{key: value}`` -> trainer flags; ``true`` becomes a bare switch, ``false`` / null are left out."""
    out: list[str] = []
    for k, v in settings.items():
        if v is True:
            out.append(f"--{k}")
        elif v is False or v is None:
            continue
        else:
            out += [f"--{k}", str(v)]
    return out


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("sweep", help="YAML file: base, common, experiments")
    ap.add_argument("--only", default=None, help="comma-separated subset of the arms")
    ap.add_argument("--gpus", type=int, default=0, help="ranks per arm (default: all GPUs of the node, 1 without GPUs)")
    ap.add_argument("--data_path", default=None, help="token file for every arm (otherwise what the base configuration says)")
    ap.add_argument("--out", default=None, help="output directory (default: outputs/sweep-<file stem>)")
    ap.add_argument("--metric", default="train/loss")
    ap.add_argument("--dry-run", action="store_true")
    argv = sys.argv[1:]
    extra: list[str] = []
    if "--" in argv:
        cut = argv.index("--")
        argv, extra = argv[:cut], argv[cut + 1:]
    a = ap.parse_args(argv)
    spec = yaml.safe_load(Path(a.sweep).read_text())
    arms: dict[str, dict[str, Any]] = spec.get("experiments") or {}
    if not arms:
        raise SystemExit(f"{a.sweep}: no experiments")
    if a.only:
        names = [n.strip() for n in a.only.split(",")]
        unknown = [n for n in names if n not in arms]
        if unknown:
            raise SystemExit(f"unknown arms {unknown}; the sweep has {list(arms)}")
        arms = {n: arms[n] for n in names}
    gpus = a.gpus or max(gpu_count(), 1)
    out = Path(a.out) if a.out else ROOT / "outputs" / f"sweep-{Path(a.sweep).stem}"
    out.mkdir(parents=True, exist_ok=True)
    shared = ["--config", str(spec["base"])] if spec.get("base") else []
    shared += flags_of(spec.get("common") or {})
    if a.data_path:
        shared += ["--data_path", a.data_path]
    records = []
    for i, (name, settings) in enumerate(arms.items()):
        d = out / name
        d.mkdir(parents=True, exist_ok=True)
        if (d / "DONE").exists() and not a.dry_run:
            print(f"\n== {name}: already done, skipped")
            records.append(json.loads((d / "DONE").read_text()))
            continue
        flags = shared + flags_of(settings or {}) + ["--checkpoint_dir", str(d), "--wandb", "--wandb_run_name", name] + extra
        rec = run_one("train", trainer_command(gpus, flags, 29700 + i), d, a.dry_run, skip=3)
        rec.update(name=name, flags=" ".join(flags))
        records.append(rec)
        if not a.dry_run and rec.get("exit_code") == 0:
            (d / "DONE").write_text(json.dumps(rec))
    if a.dry_run:
        return 0
    runs = {n: load_metrics(out / n / "metrics.jsonl") for n in arms if (out / n / "metrics.jsonl").exists()}
    runs = {n: r for n, r in runs.items() if r}
    summary: dict[str, Any] = {"sweep": str(a.sweep), "finished": datetime.datetime.now().isoformat(timespec="seconds"),
                               "gpus": gpus, "arms": records}
    if len(runs) > 1:
        cmp_ = run_analysis.compare_runs(runs, metric=a.metric)
        summary["comparison"] = cmp_
        print(f"\nranking on {a.metric}: " + " < ".join(cmp_["ranking"]))
        for n, row in cmp_["deltas"].items():
            lf = row.get("loss_final")
            if lf:
                print(f"  {n} vs {cmp_['baseline']}: final loss {lf['delta']:+.4f} ({lf['verdict']})")
    elif runs:
        summary["summary"] = {n: run_analysis.endpoint_summary(r) for n, r in runs.items()}
    (out / "sweep_summary.json").write_text(json.dumps(summary, indent=1, default=str))
    print(f"\nresults: {out}")
    return 0 if all(r.get("exit_code", 0) == 0 for r in records) else 1


if __name__ == "__main__":
    sys.exit(main())
