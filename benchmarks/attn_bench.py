#!/usr/bin/env python
"""Attention micro-benchmark: the tcgen05 flash-attention forward against PyTorch's fused SDPA
forward (library) at the 3B training shape (B=8, T=4096, 24 query / 8 kv heads, head_dim 128).

    python benchmarks/attn_bench.py [--batch 8 --seq 4096 --iters 5]
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.ops import get_ops  # noqa: E402
from kotodama_b200.ops.flash import flash_fwd  # noqa: E402


def timeit(fn, iters):
    for _ in range(2):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--heads", type=int, default=24)
    ap.add_argument("--kv", type=int, default=8)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--native-only", action="store_true")
    a = ap.parse_args()
    ops = get_ops("cuda")
    B, T, H, KV, hd = a.batch, a.seq, a.heads, a.kv, 128
    g = torch.Generator(device="cuda").manual_seed(0)
    qk = torch.randn(B * T, (H + KV) * hd, device="cuda", generator=g).bfloat16()
    qkv = torch.randn(B * T, (H + 2 * KV) * hd, device="cuda", generator=g).bfloat16()
    q, k = qk[:, : H * hd].view(B, T, H, hd), qk[:, H * hd:].view(B, T, KV, hd)
    v = qkv[:, (H + KV) * hd:].view(B, T, KV, hd)
    flops = 4.0 * B * H * T * T * hd / 2
    t_native = timeit(lambda: flash_fwd(ops, q, k, v), a.iters)
    ops.check_status()
    out = {"B": B, "T": T, "H": H, "KV": KV, "native_ms": round(t_native, 3),
           "native_tflops": round(flops / t_native / 1e9, 1)}
    if not a.native_only:
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        t_lib = timeit(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True), a.iters)
        o1, _ = flash_fwd(ops, q, k, v)
        o2 = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True).transpose(1, 2)
        out.update(sdpa_ms=round(t_lib, 3), sdpa_tflops=round(flops / t_lib / 1e9, 1), ratio=round(t_lib / t_native, 3),
                   rel_diff=float((o1.float() - o2.float()).norm() / o2.float().norm()))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
