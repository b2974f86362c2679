#!/usr/bin/env python
"""Paged decode attention alone: one new token per request against a paged KV cache, for a batch
of requests with context lengths uniform in [lo, hi]; CUDA events, L2 flushed between iterations;
achieved bytes/s against the KV bytes that must be read.

    python benchmarks/decode_attn_bench.py [--batch 64 --heads 24 --kv 8 --lo 128 --hi 2304]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.ops import get_ops  # noqa: E402


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv", type=int, default=8)
    ap.add_argument("--lo", type=int, default=128)
    ap.add_argument("--hi", type=int, default=2304)
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--splits", default="128,256,512,1024")
    ap.add_argument("--kernels", default="mma,bulk", help="of mma, bulk, stream, phases")
    a = ap.parse_args()
    ops = get_ops("cuda")
    hd, B = 128, a.batch
    g = torch.Generator(device="cuda").manual_seed(0)
    ctx = torch.randint(a.lo, a.hi + 1, (B,), device="cuda", generator=g, dtype=torch.int32)
    pages_per = (ctx + 15) // 16
    total_pages = int(pages_per.sum())
    maxp = int(pages_per.max())
    k_pages = (torch.randn(total_pages, a.kv, 16, hd, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    v_pages = (torch.randn(total_pages, a.kv, 16, hd, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    perm = torch.randperm(total_pages, device="cuda", generator=g).int()
    table = torch.zeros(B, maxp, dtype=torch.int32, device="cuda")
    o = 0
    for b in range(B):
        n = int(pages_per[b])
        table[b, :n] = perm[o:o + n]
        o += n
    q = (torch.randn(B, a.heads * hd, device="cuda", generator=g) * 0.5).to(torch.bfloat16)
    kv_bytes = float(ctx.sum()) * a.kv * hd * 2 * 2
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    max_ctx = ((int(ctx.max()) + 511) // 512) * 512
    import ctypes
    for kernel, split in [(k, int(s)) for k in a.kernels.split(",") for s in a.splits.split(",")]:
        ops.lib.kb_set_decode_kernel(ctypes.c_int({"phases": 0, "stream": 1, "bulk": 2, "mma": 3}[kernel]))
        fn = lambda: ops.paged_decode_attention(q, k_pages, v_pages, table, ctx, max_ctx, a.heads, a.kv, hd, split=split)
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        ts = []
        for _ in range(a.iters):
            flush.zero_()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record(); fn(); e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        ms = ts[len(ts) // 2]
        print(json.dumps({"kernel": kernel, "batch": B, "mean_ctx": round(float(ctx.float().mean()), 1), "split": split, "ms": round(ms, 4),
                          "kv_mb": round(kv_bytes / 1e6, 1), "gb_s": round(kv_bytes / ms / 1e6, 1)}))
    ops.check_status()


if __name__ == "__main__":
    main()
