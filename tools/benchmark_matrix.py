#!/usr/bin/env python
"""Throughput canaries and the optimisation matrix: launch the trainer under a set of configurations,
keep every log, and summarise steady-state throughput from the step lines.

    python tools/benchmark_matrix.py canary                     # 3B and 8B canaries on all GPUs of the node
    python tools/benchmark_matrix.py canary --models 8b --gpus 1
    python tools/benchmark_matrix.py matrix                     # flag matrix on configs/canary-3b.yaml
    python tools/benchmark_matrix.py matrix --config configs/proxy-benchmark.yaml --only native,nccl,fp8 --steps 60
    python tools/benchmark_matrix.py matrix --config configs/tiny-cpu.yaml --gpus 1 --only native,adamw_only   # CPU
    python tools/benchmark_matrix.py canary --dry-run           # print the commands only

Every run writes ``<out>/<name>.log`` and one record to ``<out>/results_summary.jsonl`` (exit code, wall time,
p5 / median / p95 tokens/s after the warm-up lines, device-timed tokens/s when the trainer printed it, peak
memory, last loss); ``<out>/metadata.json`` holds host, GPU, library versions and the arguments.  The canary
mode ends with wall-clock estimates for token budgets of 50-250 B at the measured rate; the matrix mode with a
table of speed-ups against the first run.  A run that fails is recorded and the others still run.

The step line the summaries are read from is ``step=... | loss=... | ... | tok/s=... | ... | gpu_mem=...GB``
(``tools/extract_benchmark_results.py``).  Counterparts of the reference's ``tools/run_canary.sh`` and
``tools/run_benchmark.sh``; the flag matrix holds this framework's switches (communication back end, fp8, tensor
parallelism, Newton-Schulz preset, ...) instead of the reference's compiler / kernel-library ones, which have no
counterpart here.
"""
from __future__ import annotations

import argparse
import datetime
import json
import os
import shlex
import socket
import subprocess
import sys
import time
from pathlib import Path
from typing import Any, Optional

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tools"))
from extract_benchmark_results import summarise  # noqa: E402

# name -> extra trainer flags; the first entry is the baseline of the speed-up column
MATRIX: dict[str, str] = {
    "native": "",
    "nccl": "--backend nccl",
    "mb8": "--micro_batch_size 8",
    "no_attnres": "--no_attn_res",
    "original_ns": "--muon_ns_coefficients original",
    "ns3": "--muon_ns_iterations 3",
    "adamw_only": "--adamw_only",
    "fp8": "--fp8",
    "tp2_sp": "--tp_size 2 --sequence_parallel",
    "tp8_sp": "--tp_size 8 --sequence_parallel",
}
TOKEN_BUDGETS = [50e9, 80e9, 100e9, 150e9, 200e9, 250e9]


def gpu_count() -> int:
    try:
        r = subprocess.run(["nvidia-smi", "-L"], capture_output=True, text=True, timeout=30)
        return len([l for l in r.stdout.splitlines() if l.startswith("GPU ")]) if r.returncode == 0 else 0
    except (OSError, subprocess.TimeoutExpired):
        return 0


def metadata(args: argparse.Namespace, runs: dict[str, list[str]]) -> dict[str, Any]:
    meta: dict[str, Any] = {"timestamp": datetime.datetime.now().isoformat(timespec="seconds"), "hostname": socket.gethostname(),
                            "gpus_used": args.gpus, "mode": args.mode, "runs": {k: " ".join(v) for k, v in runs.items()}}
    try:
        r = subprocess.run(["nvidia-smi", "--query-gpu=name,memory.total,driver_version", "--format=csv,noheader"],
                           capture_output=True, text=True, timeout=30)
        if r.returncode == 0 and r.stdout.strip():
            meta["gpu"] = r.stdout.strip().splitlines()[0]
            meta["gpu_count"] = len(r.stdout.strip().splitlines())
    except (OSError, subprocess.TimeoutExpired):
        pass
    try:
        import torch
        meta["torch_version"], meta["cuda_version"] = torch.__version__, torch.version.cuda
    except ImportError:
        pass
    return meta


def trainer_command(gpus: int, flags: list[str], port: int) -> list[str]:
    if gpus <= 1:
        return [sys.executable, str(ROOT / "train.py"), *flags]
    return [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", str(gpus), "--master-addr", "127.0.0.1",
            "--master-port", str(port), str(ROOT / "train.py"), *flags]


def run_one(name: str, cmd: list[str], out: Path, dry: bool, skip: int) -> dict[str, Any]:
    log = out / f"{name}.log"
    print(f"\n== {name}\n   {' '.join(shlex.quote(c) for c in cmd)}\n   log: {log}", flush=True)
    if dry:
        return {"name": name, "command": cmd, "dry_run": True}
    t0 = time.time()
    with open(log, "w") as fh:
        env = dict(os.environ, PYTHONUNBUFFERED="1", OMP_NUM_THREADS=os.environ.get("OMP_NUM_THREADS", "8"))
        rc = subprocess.run(cmd, stdout=fh, stderr=subprocess.STDOUT, cwd=ROOT, env=env).returncode
    rec = {"name": name, "exit_code": rc, "wall_time_s": round(time.time() - t0, 1), **summarise(str(log), skip=skip)}
    rate = rec.get("device_tok_s_median") or rec.get("tok_s_median")
    print(f"   exit {rc}, {rec['wall_time_s']} s, " + (f"{rate:,.0f} tok/s (median), " if rate else "no step lines, ")
          + f"peak memory {rec.get('gpu_mem_gb_max', 'n/a')} GB, last loss {rec.get('loss_last', 'n/a')}", flush=True)
    if rc != 0:
        print(f"   FAILED: see {log}", flush=True)
    return rec


def estimates(results: list[dict[str, Any]]) -> str:
    lines = ["", "wall-clock estimates at the measured rate:"]
    for r in results:
        rate = r.get("device_tok_s_median") or r.get("tok_s_median")
        if not rate:
            lines.append(f"  {r['name']}: no rate measured")
            continue
        lines.append(f"  {r['name']} at {rate:,.0f} tok/s (peak memory {r.get('gpu_mem_gb_max', 'n/a')} GB):")
        for b in TOKEN_BUDGETS:
            hours = b / rate / 3600
            lines.append(f"    {b / 1e9:>5.0f} B tokens -> " + (f"{hours / 24:5.1f} days ({hours:7.1f} h)" if hours >= 24 else f"{hours:5.1f} h"))
    return "\n".join(lines)


def table(results: list[dict[str, Any]]) -> str:
    rate = lambda r: r.get("device_tok_s_median") or r.get("tok_s_median")
    base: Optional[float] = next((rate(r) for r in results if rate(r)), None)
    lines = ["", f"{'run':<14}{'exit':>5}{'tok/s':>12}{'vs first':>10}{'mem GB':>9}{'loss':>9}{'wall s':>9}"]
    for r in results:
        v = rate(r)
        lines.append(f"{r['name']:<14}{r.get('exit_code', '-'):>5}{(f'{v:,.0f}' if v else '-'):>12}"
                     f"{(f'{v / base:.2f}x' if v and base else '-'):>10}{str(r.get('gpu_mem_gb_max', '-')):>9}"
                     f"{str(r.get('loss_last', '-')):>9}{str(r.get('wall_time_s', '-')):>9}")
    return "\n".join(lines)


def main() -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["canary", "matrix"])
    ap.add_argument("--models", default="3b,8b", help="canary: model sizes (configs/canary-<size>.yaml)")
    ap.add_argument("--config", default=str(ROOT / "configs" / "canary-3b.yaml"), help="matrix: base configuration")
    ap.add_argument("--only", default=None, help=f"matrix: comma-separated subset of {list(MATRIX)}")
    ap.add_argument("--gpus", type=int, default=0, help="ranks per run (default: all GPUs of the node, 1 without GPUs)")
    ap.add_argument("--steps", type=int, default=0, help="override total_steps (0: what the configuration says)")
    ap.add_argument("--skip-lines", type=int, default=3, help="step lines left out of the statistics as warm-up")
    ap.add_argument("--out", default=None, help="output directory (default: outputs/<mode>-<timestamp>)")
    ap.add_argument("--dry-run", action="store_true")
    argv = sys.argv[1:]
    extra: list[str] = []
    if "--" in argv:                                     # everything after -- goes to every trainer run
        cut = argv.index("--")
        argv, extra = argv[:cut], argv[cut + 1:]
    a = ap.parse_args(argv)
    a.gpus = a.gpus or max(gpu_count(), 1)
    out = Path(a.out) if a.out else ROOT / "outputs" / f"{a.mode}-{datetime.datetime.now():%Y%m%d-%H%M%S}"
    out.mkdir(parents=True, exist_ok=True)
    runs: dict[str, list[str]] = {}
    if a.mode == "canary":
        for size in [s.strip() for s in a.models.split(",") if s.strip()]:
            cfg = ROOT / "configs" / f"canary-{size}.yaml"
            if not cfg.exists():
                raise SystemExit(f"no canary configuration for '{size}' ({cfg})")
            runs[size] = ["--config", str(cfg)]
    else:
        names = [n.strip() for n in a.only.split(",")] if a.only else list(MATRIX)
        unknown = [n for n in names if n not in MATRIX]
        if unknown:
            raise SystemExit(f"unknown matrix entries {unknown}; choose from {list(MATRIX)}")
        for n in names:
            if n.startswith("tp") and int(n[2]) > a.gpus:
                print(f"skipping {n}: needs {n[2]} ranks, {a.gpus} in use")
                continue
            runs[n] = ["--config", a.config, *shlex.split(MATRIX[n])]
    for n in runs:
        runs[n] += ["--checkpoint_dir", str(out / f"ckpts-{n}"), "--save_every", "999999"]
        if a.steps:
            runs[n] += ["--total_steps", str(a.steps)]
        runs[n] += extra
    (out / "metadata.json").write_text(json.dumps(metadata(a, runs), indent=1))
    results = []
    with open(out / "results_summary.jsonl", "w") as summary:
        for i, (n, flags) in enumerate(runs.items()):
            rec = run_one(n, trainer_command(a.gpus, flags, 29600 + i), out, a.dry_run, a.skip_lines)
            rec["flags"] = " ".join(flags)
            summary.write(json.dumps(rec) + "\n")
            summary.flush()
            results.append(rec)
            if a.mode == "canary" and not a.dry_run:
                (out / f"{n}_summary.json").write_text(json.dumps({"model": n, "num_gpus": a.gpus, **rec}, indent=1))
    if not a.dry_run:
        print(estimates(results) if a.mode == "canary" else table(results))
    print(f"\nresults: {out}")
    return 0 if all(r.get("exit_code", 0) == 0 for r in results) else 1


if __name__ == "__main__":
    sys.exit(main())
