#!/usr/bin/env python
"""Fused GEMM+collective kernels against NCCL collectives around the same GEMM, on the
projection shapes of a model preset under tensor + sequence parallelism.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 2 --master-addr 127.0.0.1 \\
        benchmarks/tp_bench.py --model 3b --tokens 32768

Device-timed (CUDA events), warm-up, max over ranks; every iteration works on buffers far larger
than the 126 MB L2.  Prints one JSON line per case on rank 0."""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.config import MODEL_PRESETS  # noqa: E402
from kotodama_b200.ops import get_ops  # noqa: E402
from kotodama_b200.parallel.tp import TensorParallelComm, create_process_groups  # noqa: E402
from kotodama_b200.parallel.tp_native import FusedTensorParallelComm  # noqa: E402


def timed(fn, iters: int, world: int) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="3b")
    ap.add_argument("--tokens", type=int, default=32768, help="tokens of the whole TP group per micro-batch")
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--out", default="")
    args = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dist.init_process_group("nccl")
    dev = torch.device("cuda", torch.cuda.current_device())
    ops = get_ops("cuda")
    tp_group, _ = create_process_groups(world, world)
    lib = TensorParallelComm(tp_group, None, sequence_parallel=True)
    fused = FusedTensorParallelComm(tp_group, None)
    fused.setup(dev, ops)
    c = MODEL_PRESETS[args.model]
    D, F = c["hidden_size"], c["intermediate_size"]
    T, rows = args.tokens, args.tokens // world
    g = torch.Generator(device="cuda").manual_seed(rank)
    rnd = lambda *s: (torch.randn(*s, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    x_shard, w_gu = rnd(rows, D), rnd(2 * F // world, D)
    act, w_d, resid = rnd(T, F // world), rnd(D, F // world), rnd(rows, D)
    dgu, g_wgu = rnd(T, 2 * F // world), torch.zeros(2 * F // world, D, device=dev, dtype=torch.bfloat16)
    dP, g_wd = rnd(rows, D), torch.zeros(D, F // world, device=dev, dtype=torch.bfloat16)
    cases = {
        "col_linear(gate|up)  ag->gemm": lambda cm: cm.col_linear(ops, x_shard, w_gu),
        "row_linear(down)     gemm->rs": lambda cm: cm.row_linear(ops, act, w_d, residual=resid),
        "col_linear_bwd       ag->wgrad + dgrad->rs": lambda cm: cm.col_linear_bwd(ops, dgu, w_gu, x_shard, g_wgu, False),
        "row_linear_bwd       ag->dgrad + wgrad": lambda cm: cm.row_linear_bwd(ops, dP, w_d, act, g_wd, False),
    }
    rows_out = []
    for name, fn in cases.items():
        a = fn(lib).float()
        b = fn(fused).float()
        rel = float((a - b).norm() / (a.norm() + 1e-9))
        t_lib = timed(lambda: fn(lib), args.iters, world)
        t_fus = timed(lambda: fn(fused), args.iters, world)
        rec = dict(case=name, tp=world, tokens=T, nccl_ms=round(t_lib, 3), fused_ms=round(t_fus, 3),
                   speedup=round(t_lib / t_fus, 3), rel_diff=rel)
        rows_out.append(rec)
        if rank == 0:
            print(json.dumps(rec), flush=True)
    ops.check_status()
    if rank == 0 and args.out:
        with open(args.out, "w") as fh:
            for r in rows_out:
                fh.write(json.dumps(r) + "\n")
    dist.barrier()
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
