#!/usr/bin/env python
"""What AttnRes costs in a training step, by formulation of the routing.

One forward + backward of the same model is timed for

  baseline        no AttnRes: plain residual stream
  blocked         the executor's default: one phase-1 pass per block over the committed sources for all of the
                  block's queries, one phase-2 merge (fused with the RMSNorm that follows) per routing call
  per_call        every routing call is its own kernel over all its sources (``KOTODAMA_ROUTE_BLOCK_MIN`` above any block)
  module          the ``nn.Module`` forward under autograd: sources kept in Python lists and stacked at every call, the
                  formulation of the reference's training path (``src/model/llama.py:605-716``)
  blocks=N        the default formulation with N uniform blocks instead of ``--blocks`` (1 = one block for all layers,
                  L = a boundary at every layer, i.e. full attention over depth)

and the overhead of each arm over ``baseline`` is printed.  Runs on a B200 (CUDA events) and on the CPU (host clock;
``--model tiny``).  Same question as the reference's ``scripts/legacy/bench_attnres.py`` / ``bench_attnres_v2.py``, which
compare eight PyTorch formulations of the routing inside a whole model; here the arms are the formulations this framework
actually has.

    python benchmarks/attnres_step_bench.py --model 3b --micro_batch 8 --seq 4096
    python benchmarks/attnres_step_bench.py --model proxy --arms baseline,blocked,per_call,blocks=1,blocks=28
    python benchmarks/attnres_step_bench.py --model tiny --device cpu --seq 128 --json
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.engine import TrainEngine  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402


def time_calls(fn, warmup: int, iters: int, cuda: bool) -> float:
    """Median milliseconds per call: CUDA events on the device, the host clock on the CPU."""
    for _ in range(warmup):
        fn()
    ts = []
    for _ in range(iters):
        if cuda:
            torch.cuda.synchronize()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        else:
            t0 = time.perf_counter()
            fn()
            ts.append((time.perf_counter() - t0) * 1e3)
    return statistics.median(ts)


def engine_arm(a: argparse.Namespace, ids: torch.Tensor, attn_res: bool, blocks: int, block_min: int | None):
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=attn_res, attn_res_n_blocks=blocks)
    prev = os.environ.get("KOTODAMA_ROUTE_BLOCK_MIN")
    if block_min is not None:
        os.environ["KOTODAMA_ROUTE_BLOCK_MIN"] = str(block_min)
    try:
        with torch.device("meta"):
            model = KotodamaModel(cfg)
        eng = TrainEngine.from_meta(model, cfg, device=a.device, dtype=torch.bfloat16 if a.cuda else torch.float32)
    finally:
        if block_min is not None:
            if prev is None:
                os.environ.pop("KOTODAMA_ROUTE_BLOCK_MIN", None)
            else:
                os.environ["KOTODAMA_ROUTE_BLOCK_MIN"] = prev
    dev_ids = ids.to(eng.device)
    ms = time_calls(lambda: eng.forward_backward(dev_ids), a.warmup, a.iters, a.cuda)
    groups = len(eng._route_groups)
    del eng
    return ms, groups


def module_arm(a: argparse.Namespace, ids: torch.Tensor):
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=True, attn_res_n_blocks=a.blocks)
    torch.manual_seed(0)
    model = KotodamaModel(cfg).to(a.device, torch.bfloat16 if a.cuda else torch.float32)
    dev_ids = ids.to(a.device)

    def step() -> None:
        model.zero_grad(set_to_none=True)
        model(dev_ids, labels=dev_ids)["loss"].backward()
    return time_calls(step, a.warmup, a.iters, a.cuda), 0


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="proxy", choices=sorted(MODEL_PRESETS))
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--micro_batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    ap.add_argument("--blocks", type=int, default=7, help="uniform AttnRes blocks of the blocked / per_call / module arms")
    ap.add_argument("--arms", default="baseline,blocked,per_call,module")
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    a.cuda = a.device.startswith("cuda")
    layers = MODEL_PRESETS[a.model]["num_layers"]
    a.blocks = min(a.blocks, layers)
    vocab = MODEL_PRESETS[a.model]["vocab_size"]
    ids = torch.randint(0, vocab, (a.micro_batch, a.seq), generator=torch.Generator().manual_seed(0))
    rows: dict[str, dict] = {}
    for arm in [s.strip() for s in a.arms.split(",") if s.strip()]:
        if arm == "baseline":
            ms, groups = engine_arm(a, ids, False, a.blocks, None)
        elif arm == "blocked":
            ms, groups = engine_arm(a, ids, True, a.blocks, None)
        elif arm == "per_call":
            ms, groups = engine_arm(a, ids, True, a.blocks, 1 << 30)
        elif arm == "module":
            ms, groups = module_arm(a, ids)
        elif arm.startswith("blocks="):
            ms, groups = engine_arm(a, ids, True, min(int(arm.split("=", 1)[1]), layers), None)
        else:
            raise SystemExit(f"unknown arm {arm!r}")
        rows[arm] = {"ms": ms, "tokens_per_s": a.micro_batch * a.seq / (ms / 1e3), "blocked_groups": groups}
        if a.cuda:
            torch.cuda.empty_cache()
    base = rows.get("baseline", {}).get("ms")
    for r in rows.values():
        r["overhead_pct"] = None if not base else 100.0 * (r["ms"] / base - 1.0)
    if a.json:
        print(json.dumps({"model": a.model, "micro_batch": a.micro_batch, "seq": a.seq, "device": a.device, "arms": rows}))
        return
    print(f"model {a.model} ({layers} layers), {a.micro_batch} x {a.seq} tokens, forward + backward, device {a.device}")
    print(f"{'arm':<14}{'ms':>10}{'tokens/s':>12}{'vs baseline':>13}{'blocked groups':>16}")
    for arm, r in rows.items():
        ov = "" if r["overhead_pct"] is None else f"{r['overhead_pct']:+.1f}%"
        print(f"{arm:<14}{r['ms']:>10.2f}{r['tokens_per_s']:>12.0f}{ov:>13}{r['blocked_groups']:>16}")


if __name__ == "__main__":
    main()
