#!/usr/bin/env python
"""Collect the metrics of training runs in one place and summarise them.

Sources (any combination):

  positional        local run directories or ``.jsonl`` files (nothing is copied)
  --remote SPEC     ``host:path/to/checkpoint_dir`` - ``metrics.jsonl`` and ``geo_metrics.jsonl`` are
                    copied with ``scp`` (``--copy-command rsync`` uses ``rsync -az`` instead)
  --wandb PATH      ``entity/project/run_id`` - the run's full history, config and summary are
                    downloaded through the wandb API and written as ``wandb_history.jsonl`` (one
                    record per logged step, keys as logged), ``wandb_config.json``, ``wandb_summary.json``
  --list-runs E/P   list the recent runs of a wandb project and exit

    python tools/pull_metrics.py checkpoints/run-a checkpoints/run-b [--dynamics]
    python tools/pull_metrics.py --remote node2:~/ckpt/run-a -o data/pulled/run-a
    python tools/pull_metrics.py --wandb team/project/abc123 --remote node2:~/ckpt/run-a -o data/pulled/run-a

Everything pulled goes to ``--output`` (default ``data/pulled/<run>``).  Afterwards the files present are
listed with their sizes and every run gets a one-line endpoint summary (``--dynamics`` adds slopes,
plateaus and jumps; several runs are ranked by final loss).  wandb is optional: without the package the
``--wandb`` / ``--list-runs`` options say so and the rest still works.  Counterpart of the reference's
``scripts/utils/pull_metrics.py``.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
from pathlib import Path
from typing import Optional

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.eval import load_metrics, run_analysis  # noqa: E402

METRIC_FILES = ["metrics.jsonl", "geo_metrics.jsonl"]


def human(n: int) -> str:
    for unit, size in (("GB", 1 << 30), ("MB", 1 << 20), ("KB", 1 << 10)):
        if n >= size:
            return f"{n / size:.1f} {unit}"
    return f"{n} B"


def pull_remote(spec: str, out: Path, command: str = "scp", runner=subprocess.run) -> list[Path]:
    """Copy the metric files of ``host:dir``; a file the remote side does not have is skipped."""
    out.mkdir(parents=True, exist_ok=True)
    got = []
    for name in METRIC_FILES:
        src, dst = f"{spec.rstrip('/')}/{name}", out / name
        argv = ["rsync", "-az", src, str(dst)] if command == "rsync" else ["scp", "-q", src, str(dst)]
        r = runner(argv, capture_output=True, text=True)
        if r.returncode == 0 and dst.exists():
            with open(dst) as fh:
                lines = sum(1 for _ in fh)
            print(f"  {src} -> {dst} ({lines} lines)")
            got.append(dst)
        else:
            print(f"  {src}: skipped ({(r.stderr or '').strip().splitlines()[-1] if (r.stderr or '').strip() else 'not copied'})")
    return got


def pull_wandb(path: str, out: Path) -> Optional[Path]:
    """The run's history (every logged record, unsampled), config and summary."""
    try:
        import wandb
    except ImportError:
        print("  wandb is not installed: --wandb needs `pip install wandb` and WANDB_API_KEY", file=sys.stderr)
        return None
    out.mkdir(parents=True, exist_ok=True)
    run = wandb.Api().run(path)
    hist = out / "wandb_history.jsonl"
    n = 0
    with open(hist, "w") as fh:
        for row in run.scan_history():
            rec = {k: v for k, v in row.items() if v is not None and not k.startswith("_") or k == "_step"}
            if "_step" in rec:
                rec["step"] = rec.pop("_step")
            fh.write(json.dumps(rec, default=str) + "\n")
            n += 1
    (out / "wandb_config.json").write_text(json.dumps({k: v for k, v in run.config.items() if not k.startswith("_")}, indent=1, default=str))
    (out / "wandb_summary.json").write_text(json.dumps({k: v for k, v in dict(run.summary).items() if not k.startswith("_")}, indent=1, default=str))
    print(f"  {path}: {n} records -> {hist} (state {run.state}, name {run.name})")
    return hist


def list_runs(project: str) -> None:
    try:
        import wandb
    except ImportError:
        print("wandb is not installed", file=sys.stderr)
        return
    for run in wandb.Api().runs(project, order="-created_at", per_page=20):
        print(f"  {run.id:12s} {run.state:10s} {run.name}  (step {run.lastHistoryStep})")


def metrics_path(arg: str) -> Optional[Path]:
    p = Path(arg)
    if p.is_file():
        return p
    for name in METRIC_FILES + ["wandb_history.jsonl"]:
        if (p / name).is_file():
            return p / name
    return None


def summarise(runs: dict[str, Path], dynamics: bool) -> None:
    loaded = {}
    for name, path in runs.items():
        data = load_metrics(path)
        if not data:
            print(f"{name}: no records in {path}")
            continue
        loaded[name] = data
        print(json.dumps({"run": name, "file": str(path), **run_analysis.endpoint_summary(data)}))
        if dynamics:
            print(json.dumps({"run": name, "dynamics": run_analysis.training_dynamics(data)}))
    if len(loaded) > 1:
        cmp_ = run_analysis.compare_runs(loaded)
        print(json.dumps({"ranking": cmp_["ranking"], "baseline": cmp_["baseline"],
                          "loss_final_delta": {n: d.get("loss_final", {}).get("delta") for n, d in cmp_["deltas"].items()}}))


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("runs", nargs="*", help="local run directories or .jsonl files")
    ap.add_argument("--remote", "--scp", dest="remote", default=None, help="host:path/to/checkpoint_dir")
    ap.add_argument("--copy-command", choices=["scp", "rsync"], default="scp")
    ap.add_argument("--wandb", default=None, help="entity/project/run_id")
    ap.add_argument("--list-runs", default=None, metavar="ENTITY/PROJECT")
    ap.add_argument("-o", "--output", default=None, help="where pulled files go (default: data/pulled/<run>)")
    ap.add_argument("--dynamics", action="store_true", help="also print slopes, plateaus and jumps per run")
    a = ap.parse_args()
    if a.list_runs:
        list_runs(a.list_runs)
        return
    if not (a.runs or a.remote or a.wandb):
        ap.error("give local runs, --remote or --wandb")
    found: dict[str, Path] = {}
    if a.remote or a.wandb:
        label = (a.remote.rstrip("/").rsplit("/", 1)[-1] if a.remote else a.wandb.rsplit("/", 1)[-1]) or "run"
        out = Path(a.output) if a.output else Path("data/pulled") / label
        if a.wandb:
            h = pull_wandb(a.wandb, out)
            if h:
                found[f"{label} (wandb)"] = h
        if a.remote:
            got = pull_remote(a.remote, out, a.copy_command)
            if got:
                found[label] = got[0]
        if out.exists():
            print(f"pulled to {out}:")
            for f in sorted(out.iterdir()):
                print(f"  {f.name:28s} {human(f.stat().st_size)}")
    for r in a.runs:
        p = metrics_path(r)
        if p is None:
            print(f"{r}: no metrics file found", file=sys.stderr)
            continue
        found[p.parent.name if p.name in METRIC_FILES + ["wandb_history.jsonl"] else p.stem] = p
    summarise(found, a.dynamics)


if __name__ == "__main__":
    main()
