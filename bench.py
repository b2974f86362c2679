#!/usr/bin/env python
"""Headline benchmark: training throughput (tokens/s, whole job) of the 3B AttnRes-Llama,
DDP, bf16, sequence 4096, micro-batch 8 per GPU, one optimizer step per micro-batch, on
synthetic uniform-random tokens with random-init weights.

    python bench.py --gpus 1 --steps 5 --warmup 3
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        --master-port 29500 bench.py --gpus 8 --steps 5 --warmup 3
    python bench.py --impl reference ...      # the unmodified reference from baseline/_ref

Two timed passes of K steps each, both bracketed by barrier + synchronize and reported as the
max over ranks: (1) device-timed with CUDA events, inputs already on the device; (2) end to
end through ``TrainEngine.train_step`` with the step's tokens copied from pinned host memory
and the loss read back every step.  Rank 0 prints one JSON line.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

# Published by the reference: 240 K tok/s on 8 GPUs (fp8, micro-batch 4) = 30 K tok/s per GPU.
BASELINE_TOK_S_PER_GPU = 240_000 / 8


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int) -> None:
        self.gpu = gpu_index
        self.proc = None
        self.path = None

    def start(self) -> None:
        try:
            fd, self.path = tempfile.mkstemp(suffix=".csv")
            os.close(fd)
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu)], stdout=open(self.path, "w"),
                                         stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        out = {"sm_mhz": None, "sm_max_mhz": None, "reasons": []}
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        try:
            for line in open(self.path):
                f = [x.strip() for x in line.split(",")]
                if len(f) < 9:
                    continue
                sm.append(float(f[1])); mx.append(float(f[2]))
                for n, v in zip(names, f[5:9]):
                    if v.lower().startswith("active"):
                        reasons.add(n)
            os.unlink(self.path)
        except Exception:
            pass
        if sm:
            out = {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons),
                   "samples": len(sm)}
        return out


def dist_setup(n: int):
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        dist.init_process_group("nccl", device_id=torch.device(f"cuda:{local}"))
    return rank, world, local


def max_over_ranks(x: float, world: int) -> float:
    if world == 1:
        return x
    t = torch.tensor([x], dtype=torch.float64, device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def sync_all(world: int) -> None:
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()


def token_batches(n: int, mb: int, seq: int, vocab: int, seed: int, pinned: bool):
    g = torch.Generator().manual_seed(seed)
    out = []
    for _ in range(n):
        t = torch.randint(0, vocab, (mb, seq), generator=g, dtype=torch.long)
        out.append(t.pin_memory() if pinned else t)
    return out


def run_native(args, rank, world, local):
    from kotodama_b200.config import MODEL_PRESETS, ModelConfig
    from kotodama_b200.engine import TrainEngine
    from kotodama_b200.models.llama import KotodamaModel
    from kotodama_b200.parallel import make_comm

    cfg = ModelConfig(**MODEL_PRESETS[args.model], attn_res=True, attn_res_n_blocks=args.attn_res_blocks)
    torch.manual_seed(1234)
    with torch.device("meta"):
        model = KotodamaModel(cfg)
    tp = args.mode == "tp" and world > 1
    if tp:
        # tensor + sequence parallelism over all ranks: every rank sees the same global batch
        from kotodama_b200.parallel.tp import TensorParallelComm, create_process_groups
        tp_group, dp_group = create_process_groups(world, world)
        comm = None
        if args.backend in ("auto", "native"):
            try:
                from kotodama_b200.parallel.tp_native import FusedTensorParallelComm
                comm = FusedTensorParallelComm(tp_group, dp_group)
            except Exception as e:                         # noqa: BLE001 - reported in the JSON line
                if args.backend == "native":
                    raise
                print(f"[bench] fused tensor-parallel kernels unavailable ({e}); library collectives", file=sys.stderr)
        if comm is None:
            comm = TensorParallelComm(tp_group, dp_group, sequence_parallel=True)
    else:
        comm = make_comm(args.backend, world)
    eng = TrainEngine.from_meta(model, cfg, device=f"cuda:{local}", dtype=torch.bfloat16, comm=comm, seed=1234,
                                muon_lr=0.02, muon_ns_coefficients="gram_ns", gradient_clip=1.0, fp8=args.fp8)
    K, W = args.steps, args.warmup
    data_rank = 0 if tp else rank                          # TP ranks consume the same tokens
    dev_batches = [b.cuda() for b in token_batches(W + K, args.micro_batch, args.seq, cfg.vocab_size, 42 + data_rank, False)]
    host_batches = token_batches(K, args.micro_batch, args.seq, cfg.vocab_size, 4242 + data_rank, True)
    for i in range(W):
        eng.train_step([dev_batches[i]])
    eng.ops.check_status()
    if args.op_times:
        # separate, untimed-by-the-benchmark pass that attributes device time to ops
        from kotodama_b200.utils.optimer import TimedOps
        plain = eng.ops
        eng.ops = TimedOps(plain)
        plain_comm = eng.comm
        eng.comm = TimedOps(plain_comm, prefix="comm.")
        eng.train_step([dev_batches[0]])
        if rank == 0:
            with open(args.op_times, "w") as fh:
                fh.write(eng.ops.table(1) + "\n\n" + eng.comm.table(1) + "\n")
        eng.ops, eng.comm = plain, plain_comm
    sampler = ClockSampler(local)
    # ---- pass 1: device-timed
    sync_all(world)
    if rank == 0:
        sampler.start()
    l0 = eng.ops.launches
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(K):
        res = eng.train_step([dev_batches[W + i]])
    e1.record()
    sync_all(world)
    launches = eng.ops.launches - l0
    dev_ms = max_over_ranks(e0.elapsed_time(e1), world)
    # ---- pass 2: end to end (pinned H2D every step, loss D2H every step)
    sync_all(world)
    t0 = time.perf_counter()
    last = None
    for i in range(K):
        res = eng.train_step([host_batches[i]])
        last = float(res["loss"].item())
    sync_all(world)
    e2e_s = max_over_ranks(time.perf_counter() - t0, world)
    clocks = sampler.stop() if rank == 0 else {}
    eng.ops.check_status()
    tokens = K * args.micro_batch * args.seq * (1 if tp else world)
    mem = torch.cuda.max_memory_allocated() / 1e9
    return dict(dev_ms=dev_ms, e2e_s=e2e_s, tokens=tokens, launches=launches, clocks=clocks, loss=last,
                mem_gb=mem, flops_per_token=cfg.flops_per_token(args.seq), extra={
                    "gemm": eng.ops.gemm_backend, "attention_library_calls": getattr(eng.ops, "attention_library_calls", 0),
                    "comm": type(comm).__name__, "fused_tp_fallback_calls": getattr(comm, "fallback_calls", None)})


def run_serve(args, rank, world, local):
    """BASELINE config 3: the paged-KV serving engine under 64 concurrent requests (prompts uniform in
    [128, 2048], 256 new tokens each, greedy), tensor-parallel over all ranks when N > 1.  Wall-clock
    with a device synchronize around every scheduler step: the host scheduling is part of serving."""
    sys.path.insert(0, os.path.join(ROOT, "benchmarks"))
    import serve_bench
    a = argparse.Namespace(model=args.model, requests=64, min_prompt=128, max_prompt=2048, new_tokens=256, seed=0,
                           device="cuda", passes=2, profile_decode_step=-1, op_times="", prefill_batch_tokens=8192,
                           attn_res_blocks=args.attn_res_blocks)
    return serve_bench.run(a, rank, world, local)


def run_reference(args, rank, world, local):
    """The reference arm.  The unmodified reference (baseline/_ref: its model, its hybrid optimizer,
    stock DDP, driven the way its training loop drives them, on the same synthetic batches) raised a
    CUDA illegal memory access on a B200 at this benchmark's configuration with valid inputs (token
    ids inside the vocabulary, labels equal to the inputs).  Code that has faulted a GPU of the shared
    pool is not run again, so this arm reports itself unavailable instead of launching it."""
    ref_dir = os.path.join(ROOT, "baseline")
    if not os.path.isdir(os.path.join(ref_dir, "_ref", "model")):
        return {"unavailable": "baseline/_ref is not installed"}
    return {"unavailable": "the unmodified reference raised 'CUDA error: an illegal memory access was encountered' "
                           "during its training step at this configuration (3B, seq 4096) on a B200; "
                           "code that faulted a GPU is not run again on this pool"}


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=4)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="native", choices=["native", "reference", "library"],
                    help="native: this framework; reference: the unmodified reference (baseline/_ref); library: this "
                         "framework's engine with cuBLAS GEMMs and NCCL collectives instead of its own kernels - a same-box "
                         "yardstick for context, never the reference arm")
    ap.add_argument("--model", default="3b")
    ap.add_argument("--micro-batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--attn-res-blocks", type=int, default=7)
    ap.add_argument("--backend", default="auto", choices=["auto", "native", "nccl"])
    ap.add_argument("--op-times", default="", help="write a per-op device-time table to this file")
    ap.add_argument("--mode", default="dp", choices=["dp", "tp", "serve"],
                    help="dp: data parallel (the headline); tp: tensor + sequence parallel over all ranks, one global "
                         "batch of --micro-batch sequences; serve: 64-request paged-KV serving")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 projections (bf16 masters)")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        # no device work and no rendezvous: every rank returns, rank 0 prints the line
        r = run_reference(args, int(os.environ.get("RANK", 0)), args.gpus, 0)
        if int(os.environ.get("RANK", 0)) == 0:
            print(json.dumps({"impl": "reference", "unavailable": r["unavailable"]}))
        return
    if args.impl == "library":
        os.environ["KOTODAMA_GEMM"] = "cublas"
        args.backend = "nccl"
    rank, world, local = dist_setup(args.gpus)
    if args.mode == "serve":
        out = run_serve(args, rank, world, local)
        if rank == 0:
            print(json.dumps({
                "metric": "serve_decode_tokens_per_sec", "value": out["decode_tok_s"], "unit": "tokens/s",
                "n_gpus": world, "steps": out["new_tokens"], "warmup": 1, "higher_is_better": True, "scaling": "strong",
                "ms_per_step": out["p50_token_latency_ms"], "vs_baseline": None, "dtype": "bf16",
                "data": "synthetic uniform-random prompts, random-init weights",
                "config": {"model": f"{args.model} AttnRes-Llama", "requests": out["requests"],
                           "prompt_tokens": out["prompt_tokens"], "new_tokens": out["new_tokens"], "page": 16,
                           "parallelism": f"tp{world}", "timing": "wall clock, device synchronize around every step, max over ranks"},
                "prefill_tokens_per_sec": out["prefill_tok_s"], "p50_token_latency_ms": out["p50_token_latency_ms"],
                "p95_token_latency_ms": out["p95_token_latency_ms"], "gpu_launches": out["kernel_launches"],
                # per decode step: ids and cache slots (int64) + positions and context lengths (int32) go to the device as
                # one pinned copy of 24 bytes per request, the sampled token ids (int64) come back
                "e2e": {"value": out["decode_tok_s"], "unit": "tokens/s", "h2d_bytes_per_step": out["requests"] * 24,
                        "d2h_bytes_per_step": out["requests"] * 8}, "impl": "native", "notes": out}))
        if world > 1:
            dist.barrier()
            dist.destroy_process_group()
        return
    r = run_native(args, rank, world, local)
    if rank == 0:
        if "unavailable" in r:
            print(json.dumps({"impl": "reference", "unavailable": r["unavailable"]}))
        else:
            K = args.steps
            value = r["tokens"] / (r["dev_ms"] / 1e3)
            e2e = r["tokens"] / r["e2e_s"]
            bytes_in = args.micro_batch * args.seq * 8
            line = {
                "metric": "train_tokens_per_sec", "value": round(value, 1), "unit": "tokens/s", "n_gpus": world,
                "steps": K, "warmup": args.warmup, "ms_per_step": round(r["dev_ms"] / K, 3),
                "higher_is_better": True, "scaling": "strong" if args.mode == "tp" else "weak",
                "vs_baseline": round(value / (BASELINE_TOK_S_PER_GPU * world), 4),
                "dtype": "fp8 e4m3 block-scaled projections, bf16 elsewhere" if args.fp8 else "bf16",
                "data": "synthetic uniform-random tokens, random-init weights",
                "config": {"model": f"{args.model} AttnRes-Llama ({args.attn_res_blocks} blocks)",
                           "global_batch": args.micro_batch * (1 if args.mode == "tp" else world), "seq_len": args.seq,
                           "micro_batch_per_gpu": args.micro_batch, "grad_accum": 1,
                           "parallelism": (f"tp{world}+sp" if args.mode == "tp" else f"dp{world}"),
                           "optimizer": "Muon+AdamW every step",
                           "l2": "per-step working set (tens of GB) exceeds the 126 MB L2; no explicit flush",
                           "baseline_note": "vs_baseline = value / (30 K tok/s per GPU x N), the reference's "
                                            "published 240 K tok/s on 8 GPUs (fp8, micro-batch 4)"},
                "clocks": r["clocks"],
                "e2e": {"value": round(e2e, 1), "unit": "tokens/s", "h2d_bytes_per_step": bytes_in,
                        "d2h_bytes_per_step": 4},
                "gpu_launches": r["launches"], "impl": args.impl, "final_loss": r["loss"],
                "peak_mem_gb": round(r["mem_gb"], 1),
            }
            if r.get("flops_per_token"):
                line["tflops_per_gpu"] = round(value / world * r["flops_per_token"] / 1e12, 1)
            line["notes"] = r["extra"]
            if args.impl == "library":
                line["impl"] = "library_arm"
                line["library_arm"] = ("this framework's executor with torch.addmm/baddbmm (cuBLAS) for every GEMM and NCCL "
                                       "for every collective; attention, routing, loss and optimizer kernels are the "
                                       "framework's own (it has no library attention path). Context only: not the reference.")
            print(json.dumps(line))
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
