#!/usr/bin/env python
"""Serving benchmark: N concurrent requests with prompt lengths uniform in [128, 2048]
(uniform-random token ids from a seed, random-init weights), greedy decoding of 256 new tokens
each, paged KV cache with 16-token pages.  Reports prefill tok/s, decode tok/s and the p50
per-token (decode step) latency, all timed with CUDA events around the engine's steps.

    python benchmarks/serve_bench.py --model 3b --requests 64 --new-tokens 256
    python -m torch.distributed.run --nproc-per-node 8 --master-addr 127.0.0.1 benchmarks/serve_bench.py ...

Under ``torchrun`` the engine is tensor-parallel over all ranks (every rank runs the same
requests; rank 0 prints; times are the slowest rank's).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402
from kotodama_b200.models.llama import KotodamaModel  # noqa: E402
from kotodama_b200.serve.engine import SamplingParams, ServingEngine  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="3b")
    ap.add_argument("--requests", type=int, default=64)
    ap.add_argument("--new-tokens", type=int, default=256)
    ap.add_argument("--min-prompt", type=int, default=128)
    ap.add_argument("--max-prompt", type=int, default=2048)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--prefill-batch-tokens", type=int, default=8192,
                    help="rows of one padded prefill pass shared by several prompts (0: one prompt per pass)")
    ap.add_argument("--device", default="cuda")
    ap.add_argument("--passes", type=int, default=2, help="2: report the second (warm) pass, the first one separately")
    ap.add_argument("--profile-decode-step", type=int, default=-1,
                    help="bracket this decode step of the last pass with cudaProfilerStart/Stop (ncu --profile-from-start off)")
    ap.add_argument("--graph-times", action="store_true",
                    help="also report the device time of the decode graph replays alone (p50), i.e. the step without the host's share")
    ap.add_argument("--op-times", default="", help="after the run: per-op device times of 8 eager decode steps, to this file")
    a = ap.parse_args()
    world, rank = int(os.environ.get("WORLD_SIZE", "1")), int(os.environ.get("RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        if a.device == "cuda":
            torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
            dist.init_process_group("nccl", device_id=torch.device(f"cuda:{torch.cuda.current_device()}"))
        else:
            dist.init_process_group("gloo")
    out = run(a, rank, world, int(os.environ.get("LOCAL_RANK", rank)))
    if rank == 0:
        print(json.dumps(out))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


def run(a, rank: int, world: int, local: int) -> dict:
    """The benchmark proper (process group already initialised when ``world > 1``); returns the result
    dictionary on every rank (times are the slowest rank's)."""
    cuda = a.device.startswith("cuda")
    tp = None
    if world > 1:
        from kotodama_b200.serve.tp import ServeTP
        if cuda:
            a.device = f"cuda:{torch.cuda.current_device()}"
        tp = ServeTP()
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=True, attn_res_n_blocks=7 if a.model != "tiny" else 2)
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    eng = ServingEngine(model, device=a.device, dtype=torch.bfloat16 if cuda else torch.float32,
                        max_batch=a.requests, max_ctx=a.max_prompt + a.new_tokens + 16, tp=tp,
                        prefill_batch_tokens=a.prefill_batch_tokens)
    eng.arena.init_weights(cfg.num_layers, a.seed)
    g = torch.Generator().manual_seed(a.seed)
    lens = torch.randint(a.min_prompt, a.max_prompt + 1, (a.requests,), generator=g).tolist()
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in lens]
    # warm-up on a short request (kernel attribute setup, allocator)
    eng.generate([prompts[0][:64]], SamplingParams(max_new_tokens=4, temperature=0.0))
    sync = torch.cuda.synchronize if cuda else (lambda: None)
    import time

    def one_pass(profile_step: int = -1):
        """The whole workload once: admit + prefill all requests, decode to completion."""
        before = dict(eng.stats)
        reqs = [eng.add_request(p, SamplingParams(max_new_tokens=a.new_tokens, temperature=0.0)) for p in prompts]
        sync()
        t0 = time.perf_counter()
        eng.step()                       # admits and prefills every request, then one decode step
        sync()
        t_first = time.perf_counter() - t0
        print(f"[rank {rank}] prefill + first step done in {t_first:.2f}s", file=sys.stderr, flush=True)
        step_ms = []
        while eng.has_work():
            sync()
            prof = cuda and len(step_ms) == profile_step
            if prof:
                torch.cuda.profiler.start()
            t = time.perf_counter()
            eng.step()
            sync()
            step_ms.append((time.perf_counter() - t) * 1e3)
            if prof:
                torch.cuda.profiler.stop()
        decode_tokens = sum(len(r.generated) for r in reqs) - 2 * len(reqs)   # minus prefill token and first step
        return dict(t_first=t_first, step_ms=step_ms, decode_tokens=decode_tokens,
                    prefill_s=eng.stats["prefill_s"] - before["prefill_s"])

    if cuda and a.graph_times:
        eng.graph_ms = []
    cold = one_pass()                    # first pass: allocator growth, graph capture, first-use set-up
    res = one_pass(a.profile_decode_step) if a.passes > 1 else cold
    t_first, step_ms, decode_tokens = res["t_first"], res["step_ms"], res["decode_tokens"]
    if a.op_times and cuda:
        # a second, eager pass (no graphs) over a few decode steps with every op bracketed by events
        from kotodama_b200.utils.optimer import TimedOps
        eng.use_cuda_graphs = False
        plain = eng.ops
        eng.ops = TimedOps(plain)
        for p_ in prompts[:16]:
            eng.add_request(p_, SamplingParams(max_new_tokens=12, temperature=0.0))
        sync()
        t = time.perf_counter()
        eng.step()                   # 16 prefills + one decode step
        sync()
        wall_prefill = time.perf_counter() - t
        table_prefill = eng.ops.table(1)
        eng.ops.reset()
        n_steps = 0
        sync()
        t = time.perf_counter()
        while eng.has_work() and n_steps < 8:
            eng.step()
            n_steps += 1
        sync()
        wall_decode = (time.perf_counter() - t) / max(n_steps, 1)
        if rank == 0:
            with open(a.op_times, "w") as fh:
                fh.write(f"== 16 prefills ({sum(lens[:16])} tokens) + 1 decode step, eager: wall {wall_prefill * 1e3:.1f} ms\n")
                fh.write(table_prefill + "\n\n")
                fh.write(f"== decode step (batch 16), eager, mean of {n_steps}: wall {wall_decode * 1e3:.2f} ms\n")
                fh.write(eng.ops.table(max(n_steps, 1)) + "\n")
        eng.ops = plain
        while eng.has_work():
            eng.step()
    total_decode_s = sum(step_ms) / 1e3
    out = {"model": a.model, "requests": a.requests, "prompt_tokens": sum(lens), "new_tokens": a.new_tokens,
           "prefill_plus_first_step_s": round(t_first, 3),
           "prefill_tok_s": round(sum(lens) / max(res["prefill_s"], 1e-9), 1),
           "first_pass": {"prefill_tok_s": round(sum(lens) / max(cold["prefill_s"], 1e-9), 1),
                          "decode_tok_s": round(cold["decode_tokens"] / max(sum(cold["step_ms"]) / 1e3, 1e-9), 1)},
           "decode_tok_s": round(decode_tokens / max(total_decode_s, 1e-9), 1),
           "p50_token_latency_ms": round(statistics.median(step_ms), 3) if step_ms else None,
           "p95_token_latency_ms": round(sorted(step_ms)[int(0.95 * (len(step_ms) - 1))], 3) if step_ms else None,
           "decode_graph_ms_p50": (round(statistics.median(eng.graph_ms[-len(step_ms):]), 3)
                                   if eng.graph_ms and step_ms else None),
           "kernel_launches": getattr(eng.ops, "launches", None),
           "attention_library_calls": getattr(eng.ops, "attention_library_calls", 0), "tp": world,
           "prefill_passes": eng.stats["prefill_passes"], "prefill_batch_tokens": a.prefill_batch_tokens}
    if tp is not None:
        out.update(native_allreduce_calls=tp.native_calls, library_allreduce_calls=tp.library_calls,
                   multimem_allreduce_calls=tp.multimem_calls, fused_gemm_allreduce_calls=tp.fused_calls)
    if hasattr(eng.ops, "check_status"):
        eng.ops.check_status()
    if tp is not None:
        import torch.distributed as dist
        t = torch.tensor([out["prefill_plus_first_step_s"], total_decode_s, statistics.median(step_ms)],
                         dtype=torch.float64, device=a.device if cuda else "cpu")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["prefill_plus_first_step_s"] = round(float(t[0]), 3)
        out["decode_tok_s"] = round(decode_tokens / max(float(t[1]), 1e-9), 1)
        out["p50_token_latency_ms"] = round(float(t[2]), 3)
    return out


if __name__ == "__main__":
    main()
