#!/usr/bin/env python
"""Where one training step spends its time, on one device, three views:

1. phases (CUDA events around the executor's calls): forward + backward, optimizer step, whole step;
2. ops (every op of the executor bracketed by events, one extra step): GEMMs, attention, routing,
   cross-entropy, Newton-Schulz, AdamW, ... with call counts and shares;
3. kernels (``--trace out.json``): a ``torch.profiler`` trace of ``--profile_steps`` steps, exported for
   chrome://tracing / Perfetto and summarised by kernel name (``tools/parse_profile.py`` reads the same file).

    python tools/profile_step.py --model proxy --micro_batch 4 --seq 2048
    python tools/profile_step.py --model 3b --micro_batch 8 --seq 4096 --optimizer adamw
    python tools/profile_step.py --model proxy --ns_iter 3 --trace /tmp/step.json --profile_steps 2
    python tools/profile_step.py --model tiny --device cpu --seq 128

``--optimizer muon`` (default) runs the hybrid Muon + AdamW step, ``adamw`` the AdamW-only arm; ``--ns_iter`` sets the
Newton-Schulz iterations of Muon; ``--fp8`` runs the projections in block-scaled fp8.  There is no tracing compiler
in this framework, so the reference tool's ``--compile`` switch has no counterpart.  Counterpart of the reference's
``scripts/utils/profile_step.py``.
"""
from __future__ import annotations

import argparse
import os
import sys
from collections import defaultdict

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.monitor.profiler import PhaseTimer  # noqa: E402
from kotodama_b200.utils.optimer import TimedOps  # noqa: E402


def build_engine(a: argparse.Namespace, dev: str) -> tuple[TrainEngine, ModelConfig]:
    small = a.model in ("tiny", "smoke")
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=not a.no_attn_res, attn_res_n_blocks=2 if small else a.attn_res_n_blocks)
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    eng = TrainEngine.from_meta(model, cfg, device=dev, dtype=torch.bfloat16 if dev.startswith("cuda") else torch.float32,
                                adamw_only=a.optimizer == "adamw", muon_ns_iterations=a.ns_iter, fp8=a.fp8)
    return eng, cfg


def kernel_table(prof, steps: int, top: int = 30) -> str:
    """Device time per kernel name over the traced steps."""
    tot, cnt = defaultdict(float), defaultdict(int)
    for e in prof.events():
        t = getattr(e, "device_time_total", 0.0)
        if t and e.device_type.name != "CPU":
            tot[e.name] += t
            cnt[e.name] += 1
    if not tot:
        return "(no device kernels in the trace)"
    total = sum(tot.values())
    rows = sorted(tot.items(), key=lambda kv: -kv[1])[:top]
    lines = [f"{'kernel':<80}{'ms/step':>10}{'calls/step':>12}{'share':>8}"]
    for name, t in rows:
        lines.append(f"{name[:78]:<80}{t / 1e3 / steps:>10.3f}{cnt[name] / steps:>12.1f}{100 * t / total:>7.1f}%")
    lines.append(f"{'total traced device time':<80}{total / 1e3 / steps:>10.3f}")
    return "\n".join(lines)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="proxy", choices=sorted(MODEL_PRESETS))
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--micro_batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--optimizer", choices=["muon", "adamw"], default="muon")
    ap.add_argument("--muon", dest="optimizer", action="store_const", const="muon", help="same as --optimizer muon")
    ap.add_argument("--adamw", dest="optimizer", action="store_const", const="adamw", help="same as --optimizer adamw")
    ap.add_argument("--ns_iter", type=int, default=5)
    ap.add_argument("--fp8", action="store_true")
    ap.add_argument("--no_attn_res", action="store_true")
    ap.add_argument("--attn_res_n_blocks", type=int, default=7)
    ap.add_argument("--warmup_steps", type=int, default=2)
    ap.add_argument("--steps", "--profile_steps", dest="steps", type=int, default=3)
    ap.add_argument("--compile", action="store_true", help="accepted for command-line compatibility; there is no tracing compiler here")
    ap.add_argument("--trace", default=None, help="also record a torch.profiler trace of the timed steps to this file")
    a = ap.parse_args()
    dev = a.device
    eng, cfg = build_engine(a, dev)
    ids = torch.randint(0, cfg.vocab_size, (a.micro_batch, a.seq))
    for _ in range(a.warmup_steps):
        eng.train_step([ids])
    print(f"model {a.model}, {a.micro_batch} x {a.seq} tokens, optimizer {a.optimizer}, ns_iter {a.ns_iter}, device {dev}")
    # ---- 1. phases
    timer = PhaseTimer(dev.startswith("cuda"))
    for _ in range(a.steps):
        with timer.phase("FULL_STEP"):
            with timer.phase("FORWARD_BACKWARD"):
                eng.forward_backward(ids.to(eng.device))
            with timer.phase("OPTIMIZER_STEP"):
                eng.optimizer_step()
    totals = timer.totals_ms()
    full = totals.get("FULL_STEP", 0.0) / a.steps
    print("\n== phases")
    for k, v in totals.items():
        print(f"{k:<20}{v / a.steps:>10.2f} ms/step{100 * v / a.steps / full if full else 0:>8.1f}%")
    if full:
        print(f"{'tokens/s':<20}{a.micro_batch * a.seq / (full / 1e3):>10.0f}")
    # ---- 2. ops
    plain = eng.ops
    eng.ops = TimedOps(plain)
    eng.train_step([ids])
    print("\n== ops (one step, every op bracketed by events)")
    print(eng.ops.table(1))
    eng.ops = plain
    # ---- 3. kernels
    if a.trace:
        from torch.profiler import ProfilerActivity, profile
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if dev.startswith("cuda") else [])
        with profile(activities=acts) as prof:
            for _ in range(a.steps):
                eng.train_step([ids])
            if dev.startswith("cuda"):
                torch.cuda.synchronize()
        prof.export_chrome_trace(a.trace)
        print(f"\n== kernels ({a.steps} steps, trace -> {a.trace})")
        print(kernel_table(prof, a.steps))


if __name__ == "__main__":
    main()
