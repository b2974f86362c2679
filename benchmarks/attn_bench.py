#!/usr/bin/env python
"""Attention micro-benchmark: the tcgen05 flash-attention forward and backward against PyTorch's
fused SDPA (a library kernel, used here only as the yardstick) at the 3B training shape (B=8,
T=4096, 24 query / 8 kv heads, head_dim 128).

    python benchmarks/attn_bench.py [--batch 8 --seq 4096 --iters 5] [--native-only] [--fwd-only]
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
from kotodama_b200.ops.flash import flash_bwd, flash_fwd  # noqa: E402


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
    ap.add_argument("--fwd-only", action="store_true")
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
    do = torch.randn(B, T, H, hd, device="cuda", generator=g).bfloat16()
    if not a.fwd_only:
        o, lse = flash_fwd(ops, q, k, v)
        dqk, dqkv = torch.empty_like(qk), torch.empty_like(qkv)
        dq, dk = dqk[:, : H * hd].view(B, T, H, hd), dqk[:, H * hd:].view(B, T, KV, hd)
        dv = dqkv[:, (H + KV) * hd:].view(B, T, KV, hd)
        t_bwd = timeit(lambda: flash_bwd(ops, do, q, k, v, o, lse, dq, dk, dv), a.iters)
        t_kv = timeit(lambda: flash_bwd(ops, do, q, k, v, o, lse, dq, dk, dv, which=1), a.iters)
        t_q = timeit(lambda: flash_bwd(ops, do, q, k, v, o, lse, dq, dk, dv, which=2), a.iters)
        ops.check_status()
        out.update(native_bwd_ms=round(t_bwd, 3), native_bwd_tflops=round(2.5 * flops / t_bwd / 1e9, 1),
                   native_dkdv_ms=round(t_kv, 3), native_dq_ms=round(t_q, 3))
    if not a.native_only:
        qt, kt, vt = q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2)
        t_lib = timeit(lambda: F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True), a.iters)
        o1, _ = flash_fwd(ops, q, k, v)
        o2 = F.scaled_dot_product_attention(qt, kt, vt, is_causal=True, enable_gqa=True).transpose(1, 2)
        out.update(sdpa_ms=round(t_lib, 3), sdpa_tflops=round(flops / t_lib / 1e9, 1), ratio=round(t_lib / t_native, 3),
                   rel_diff=float((o1.float() - o2.float()).norm() / o2.float().norm()))
        if not a.fwd_only:
            ql, kl, vl = (x.detach().clone().requires_grad_(True) for x in (qt, kt, vt))
            ol = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=True)
            dot = do.transpose(1, 2)
            t_lb = timeit(lambda: torch.autograd.grad(ol, (ql, kl, vl), dot, retain_graph=True), a.iters)
            gq, gk, gv = torch.autograd.grad(ol, (ql, kl, vl), dot, retain_graph=True)
            rd = lambda x, y: float((x.float() - y.float()).norm() / y.float().norm())
            out.update(sdpa_bwd_ms=round(t_lb, 3), sdpa_bwd_tflops=round(2.5 * flops / t_lb / 1e9, 1),
                       bwd_ratio=round(t_lb / t_bwd, 3), dq_diff=rd(dq, gq.transpose(1, 2)),
                       dk_diff=rd(dk, gk.transpose(1, 2)), dv_diff=rd(dv, gv.transpose(1, 2)))
    print(json.dumps(out))


if __name__ == "__main__":
    main()
