#!/usr/bin/env python
"""GEMM micro-benchmark: the tcgen05 kernel against cuBLAS (torch.matmul) on the projection
shapes of the 3B/8B models, for the forward (NT), data-gradient (NN) and weight-gradient (TN)
products.  CUDA events, warm-up, L2 flushed between iterations.

    python benchmarks/gemm_bench.py                       # table for the 3B shapes
    python benchmarks/gemm_bench.py --single 4096 8192 3072 nt --iters 3   # small case for ncu
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from kotodama_b200.ops import get_ops  # noqa: E402


def time_fn(fn, iters: int, flush: torch.Tensor) -> float:
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush.zero_()                    # 256 MB write: evicts the 126 MB L2
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def operands(M, N, K, mode, dtype=torch.bfloat16):
    g = torch.Generator(device="cuda").manual_seed(0)
    r = lambda *s: (torch.randn(*s, device="cuda", generator=g) * 0.05).to(dtype)
    if mode == "nt":
        return r(M, K), r(N, K)
    if mode == "nn":
        return r(M, K), r(K, N)
    return r(K, M), r(K, N)


def run(ops, M, N, K, mode, iters, flush):
    a, b = operands(M, N, K, mode)
    out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
    mine = {"nt": lambda: ops.gemm_nt(a, b, out=out), "nn": lambda: ops.gemm_nn(a, b, out=out),
            "tn": lambda: ops.gemm_tn(a, b, out=out)}[mode]
    lib = {"nt": lambda: torch.matmul(a, b.t(), out=out), "nn": lambda: torch.matmul(a, b, out=out),
           "tn": lambda: torch.matmul(a.t(), b, out=out)}[mode]
    t_mine = time_fn(mine, iters, flush)
    ref = out.clone().float()
    t_lib = time_fn(lib, iters, flush)
    err = float((out.float() - ref).norm() / (out.float().norm() + 1e-9))
    fl = 2.0 * M * N * K
    return dict(M=M, N=N, K=K, mode=mode, ms=round(t_mine, 4), tflops=round(fl / t_mine / 1e9, 1),
                cublas_ms=round(t_lib, 4), cublas_tflops=round(fl / t_lib / 1e9, 1),
                ratio=round(t_lib / t_mine, 3), rel_diff=err)


def fp8_table(ops, args, flush) -> None:
    """Forward-shaped products of the preset: fp8 GEMM alone, with the activation quantiser, and the
    bf16 tcgen05 GEMM / cuBLAS on the same shape."""
    from kotodama_b200.config import MODEL_PRESETS
    c = MODEL_PRESETS[args.model]
    D, F = c["hidden_size"], c["intermediate_size"]
    QKV = (c["num_attention_heads"] + 2 * c["num_kv_heads"]) * c["head_dim"]
    T = args.tokens
    shapes = [(T, QKV, D), (T, D, c["num_attention_heads"] * c["head_dim"]), (T, 2 * F, D), (T, D, F)]
    if args.single:
        shapes = [tuple(map(int, args.single[:3]))]
    for (M, N, K) in shapes:
        a, b = operands(M, N, K, "nt")
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        # the other back end first (for the record), then the selected one
        chosen = ops.fp8_backend
        other = "promote" if chosen == "mx" else "mx"
        ops.fp8_backend, ops.fp8_pow2 = other, other == "mx"
        qa, sa = ops.quant_rows(a)
        qb, sb = ops.quant_blocks(b)
        t_other = time_fn(lambda: ops.gemm_fp8(qa, sa, qb, sb, 128, out=out), args.iters, flush)
        ops.fp8_backend, ops.fp8_pow2 = chosen, chosen == "mx"
        qa, sa = ops.quant_rows(a)
        qb, sb = ops.quant_blocks(b)
        t_g = time_fn(lambda: ops.gemm_fp8(qa, sa, qb, sb, 128, out=out), args.iters, flush)
        t_q = time_fn(lambda: ops.quant_rows(a), args.iters, flush)
        qat, sat = ops.quant_cols_t(a)
        t_w = time_fn(lambda: ops.gemm_fp8(qat[:, :], sat, qat, sat, 1), 3, flush) if M % 128 == 0 and args.single else 0.0
        t_b = time_fn(lambda: ops.gemm_nt(a, b, out=out), args.iters, flush)
        t_l = time_fn(lambda: torch.matmul(a, b.t(), out=out), args.iters, flush)
        fl = 2.0 * M * N * K
        print(json.dumps(dict(M=M, N=N, K=K, backend=chosen, fp8_ms=round(t_g, 4), fp8_tflops=round(fl / t_g / 1e9, 1),
                              **{f"{other}_ms": round(t_other, 4)},
                              quant_rows_ms=round(t_q, 4), quant_gbs=round(M * K * 3 / t_q / 1e6, 1),
                              bf16_ms=round(t_b, 4), cublas_bf16_ms=round(t_l, 4),
                              fp8_vs_bf16=round(t_b / t_g, 3), fp8_plus_quant_vs_bf16=round(t_b / (t_g + t_q), 3))))
    ops.check_status()


def decode_table(ops, args) -> None:
    """The four projections of a decode step (M = --decode-rows) for every layer of the preset, timed inside a
    CUDA graph (distinct weights per layer, so every product streams its weight from memory): the cluster
    split-K kernel, split-K with fp32 atomics + finishing kernel, and cuBLAS (torch.addmm)."""
    from kotodama_b200.config import MODEL_PRESETS
    c = MODEL_PRESETS[args.model]
    D, F, L = c["hidden_size"], c["intermediate_size"], c["num_layers"]
    QKV = (c["num_attention_heads"] + 2 * c["num_kv_heads"]) * c["head_dim"]
    shapes = [(QKV, D), (D, c["num_attention_heads"] * c["head_dim"]), (2 * F, D), (D, F)]
    M = args.decode_rows
    g = torch.Generator(device="cuda").manual_seed(0)
    r = lambda *s_: (torch.randn(*s_, device="cuda", generator=g) * 0.05).to(torch.bfloat16)
    ws = [[r(N, K) for (N, K) in shapes] for _ in range(L)]
    acts = {K: r(M, K) for (_, K) in shapes}
    res = {N: r(M, N) for (N, _) in shapes}

    def mine():
        for l in range(L):
            for i, (N, K) in enumerate(shapes):
                ops.gemm_nt(acts[K], ws[l][i], residual=res[N])

    def lib():
        for l in range(L):
            for i, (N, K) in enumerate(shapes):
                torch.addmm(res[N], acts[K], ws[l][i].t())

    def graph_ms(fn):
        fn()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            fn()
        for _ in range(3):
            gr.replay()
        torch.cuda.synchronize()
        ts = []
        for _ in range(max(args.iters, 1)):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            gr.replay()
            e1.record()
            torch.cuda.synchronize()
            ts.append(e0.elapsed_time(e1))
        ts.sort()
        return ts[len(ts) // 2]
    by = sum(N * K * 2 for N, K in shapes) * L
    arms = [("cluster split-K (DSMEM)", True, mine), ("split-K atomics + finish", False, mine), ("cuBLAS addmm", None, lib)]
    for name, cluster, fn in arms:
        if cluster is not None:
            ops.skinny_cluster = cluster
        ms = graph_ms(fn)
        print(json.dumps({"arm": name, "rows": M, "products": 4 * L, "ms_per_step": round(ms, 3),
                          "weight_TBs": round(by / ms / 1e9, 2), "ideal_ms": round(by / 6451.8e6, 3)}))
    ops.skinny_cluster = True
    ops.check_status()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--single", nargs=4, default=None, metavar=("M", "N", "K", "MODE"))
    ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--tokens", type=int, default=32768)
    ap.add_argument("--model", default="3b")
    ap.add_argument("--out", default="")
    ap.add_argument("--two-cta", type=int, default=-1, help="force the CTA-pair kernel on (1) or off (0)")
    ap.add_argument("--fp8", action="store_true", help="block-scaled e4m3 GEMM (quantisation timed separately)")
    ap.add_argument("--decode", action="store_true", help="decode-size products of every layer inside a CUDA graph")
    ap.add_argument("--decode-rows", type=int, default=64)
    args = ap.parse_args()
    ops = get_ops("cuda")
    if args.two_cta >= 0:
        ops.gemm_2cta = bool(args.two_cta)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    if args.fp8:
        fp8_table(ops, args, flush)
        return
    if args.decode:
        decode_table(ops, args)
        return
    if args.single:
        M, N, K = map(int, args.single[:3])
        a, b = operands(M, N, K, args.single[3])
        out = torch.empty(M, N, device="cuda", dtype=torch.bfloat16)
        fn = {"nt": ops.gemm_nt, "nn": ops.gemm_nn, "tn": ops.gemm_tn}[args.single[3]]
        for _ in range(args.iters):
            fn(a, b, out=out)
        torch.cuda.synchronize()
        ops.check_status()
        print("ok")
        return
    from kotodama_b200.config import MODEL_PRESETS
    c = MODEL_PRESETS[args.model]
    D, F = c["hidden_size"], c["intermediate_size"]
    QKV = (c["num_attention_heads"] + 2 * c["num_kv_heads"]) * c["head_dim"]
    Q = c["num_attention_heads"] * c["head_dim"]
    T = args.tokens
    shapes = []
    for (n, k) in ((QKV, D), (D, Q), (2 * F, D), (D, F)):
        shapes += [(T, n, k, "nt"), (T, k, n, "nn"), (n, k, T, "tn")]
    shapes += [(4096, c["vocab_size"], D, "nt"), (4096, D, c["vocab_size"], "nn"), (c["vocab_size"], D, 4096, "tn")]
    rows = [run(ops, *s, args.iters, flush) for s in shapes]
    ops.check_status()
    for r in rows:
        print(json.dumps(r))
    tot_m = sum(r["ms"] for r in rows)
    tot_l = sum(r["cublas_ms"] for r in rows)
    print(json.dumps({"total_ms": round(tot_m, 3), "cublas_total_ms": round(tot_l, 3), "ratio": round(tot_l / tot_m, 3)}))
    if args.out:
        with open(args.out, "w") as fh:
            for r in rows:
                fh.write(json.dumps(r) + "\n")


if __name__ == "__main__":
    main()
