#!/usr/bin/env python
"""AttnRes routing + RMSNorm micro-benchmark: achieved HBM bandwidth of the fused forward and
backward kernels for S = 1..8 sources against a plain device copy of the same byte count.

    python benchmarks/route_bench.py                         # table (3B shape: N=32768, D=3072)
    python benchmarks/route_bench.py --single 8 --tokens 8192 --iters 2     # small case for ncu
    python benchmarks/route_bench.py --blocked [--single 7 --queries 8]    # the blocked kernels (phase 1 / phase 2)
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.ops import get_ops  # noqa: E402


def make(N, D, S):
    g = torch.Generator(device="cuda").manual_seed(0)
    srcs = [(torch.randn(N, D, device="cuda", generator=g)).bfloat16() for _ in range(S)]
    q = (torch.randn(D, device="cuda", generator=g) * 0.3).bfloat16()
    rn = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    nw = torch.ones(D, device="cuda", dtype=torch.bfloat16)
    dxn = torch.randn(N, D, device="cuda", generator=g).bfloat16()
    ds = [torch.zeros(N, D, device="cuda", dtype=torch.bfloat16) for _ in range(S)]
    return srcs, q, rn, nw, dxn, ds


def timeit(fn, iters):
    fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); fn(); e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    return sorted(ts)[len(ts) // 2]


def blocked(ops, a, N, D, row):
    """Phase-1 (Q queries over S committed sources) and phase-2 (one query, partial merge + RMSNorm)
    kernels, forward and backward, with the bytes each must move."""
    Q = a.queries
    g = torch.Generator(device="cuda").manual_seed(0)
    for S in ([a.single] if a.single else [2, 4, 7]):
        srcs, q, rn, nw, dxn, ds = make(N, D, S)
        qs = (torch.randn(Q, D, device="cuda", generator=g) * 0.3).bfloat16()
        rns = torch.ones(Q, D, device="cuda", dtype=torch.bfloat16)
        st = {}
        def p1f():
            st["p1"] = ops.route_p1_fwd(srcs, qs, rns, 1e-5)
        t1f = timeit(p1f, a.iters)
        o, lse, stats = st["p1"]
        part = torch.randn(N, D, device="cuda", generator=g).bfloat16()
        def p2f():
            st["p2"] = ops.route_p2_fwd(o[1], lse[1], part, q, rn, nw, 1e-5)
        t2f = timeit(p2f, a.iters)
        do, dlse = torch.empty_like(o), torch.empty_like(lse)
        dpart = torch.zeros_like(part)
        t2b = timeit(lambda: ops.route_p2_bwd(dxn, o[1], lse[1], part, q, rn, nw, 1e-5, st["p2"][1], do[1], dlse[1],
                                              dpart, True), a.iters)
        do.normal_(generator=g)
        dlse.normal_(generator=g)
        t1b = timeit(lambda: ops.route_p1_bwd(srcs, qs, rns, do, dlse, lse, stats, ds, [True] * S), a.iters)
        gb = lambda rows, ms: round(rows * row / ms / 1e6, 1)
        print(json.dumps({"S": S, "Q": Q, "N": N, "D": D,
                          "p1_fwd_ms": round(t1f, 3), "p1_fwd_GBs": gb(S + Q, t1f),
                          "p2_fwd_ms": round(t2f, 3), "p2_fwd_GBs": gb(3, t2f),
                          "p2_bwd_ms": round(t2b, 3), "p2_bwd_GBs": gb(6, t2b),
                          "p1_bwd_ms": round(t1b, 3), "p1_bwd_GBs": gb(3 * S + Q, t1b)}))
    ops.check_status()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--dim", type=int, default=3072)
    ap.add_argument("--iters", type=int, default=5)
    ap.add_argument("--single", type=int, default=0)
    ap.add_argument("--blocked", action="store_true")
    ap.add_argument("--queries", type=int, default=8)
    a = ap.parse_args()
    ops = get_ops("cuda")
    N, D = a.tokens, a.dim
    row = N * D * 2
    if a.blocked:
        return blocked(ops, a, N, D, row)
    for S in ([a.single] if a.single else [1, 2, 4, 6, 8]):
        srcs, q, rn, nw, dxn, ds = make(N, D, S)
        st = {}
        def fwd():
            st["o"] = ops.route_norm_fwd(srcs, q, rn, nw, 1e-5)
        def bwd():
            ops.route_norm_bwd(dxn, srcs, q, rn, nw, 1e-5, st["o"][1], ds, [True] * S)
        tf = timeit(fwd, a.iters)
        tb = timeit(bwd, a.iters)
        big = torch.empty((S + 1) * N * D, device="cuda", dtype=torch.bfloat16)
        dst = torch.empty_like(big)
        tc = timeit(lambda: dst.copy_(big), a.iters)
        fb, bb = (S + 1) * row, (3 * S + 1) * row
        print(json.dumps({"S": S, "N": N, "D": D, "fwd_ms": round(tf, 3), "fwd_GBs": round(fb / tf / 1e6, 1),
                          "bwd_ms": round(tb, 3), "bwd_GBs": round(bb / tb / 1e6, 1),
                          "copy_GBs": round(2 * (S + 1) * row / tc / 1e6, 1)}))
        del big, dst
    ops.check_status()


if __name__ == "__main__":
    main()
