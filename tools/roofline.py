#!/usr/bin/env python
"""Lower bounds for a training step and a decode step from the model's shapes and the machine's measured peaks.

Every op of a step is either a product (bounded by FLOPs / tensor-core peak) or a streaming pass (bounded by
bytes / memory bandwidth); the step's floor is the sum of the per-op bounds, and the communication floor (bytes that
must cross NVLink / link bandwidth) is printed beside it because it overlaps with compute.  With ``--measured_ms`` the
achieved fraction is printed, which is how the roofline fractions of the measurement tables are obtained.

    python tools/roofline.py train --model 3b --micro_batch 8 --seq 4096 [--gpus 8] [--tp 8] [--measured_ms 714.3]
    python tools/roofline.py decode --model 3b --batch 64 --context 1220 [--tp 8] [--measured_ms 4.31]
    python tools/roofline.py train --model 8b --micro_batch 4 --seq 4096 --blocks 8 --json

Peaks are read from a JSON file (``--peaks``, default ``MEASURED_PEAKS.json`` beside the package: ``hbm_gbs``,
``bf16_tflops_sustained``); without one the nominal B200 figures are used and said so.  What is counted:

* products: ``6 x parameters-in-products x tokens`` (forward, data gradient, weight gradient) and causal attention
  (two products forward, five backward with the recomputed scores, half of each square; the throughput figures of
  the benchmarks count four backward products, i.e. they do not credit the recomputation);
* Newton-Schulz: per matrix of m x n (m <= n) and iteration, ``X X^T`` and ``A A`` over the upper triangle only and
  ``B X`` in full: ``(m^2 n + m^3 + 2 m^2 n)`` FLOPs, matrices divided over the data-parallel ranks that own them;
* streaming passes (bf16 activations): AttnRes routing in blocked form (every committed source is read once per block
  in each direction, every routing call reads and writes a handful of token-major tensors), RMSNorm, QK-norm + RoPE,
  SwiGLU, the chunked loss head (logits written once and re-read, then
  written and re-read as gradient), and the optimizer (parameter, gradient and moments per element);
* decode: every weight and every cached key / value of the batch is read once per step.
"""
from __future__ import annotations

import argparse
import json
import os
import sys
from typing import Any

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.config import MODEL_PRESETS, ModelConfig  # noqa: E402

NOMINAL = {"hbm_gbs": 7700.0, "bf16_tflops_sustained": 2250.0, "source": "nominal B200 figures"}
NVLINK_GBS = 770.0            # measured peer copy, per direction per GPU


def load_peaks(path: str | None) -> dict[str, Any]:
    cand = path or os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "MEASURED_PEAKS.json")
    if os.path.exists(cand):
        with open(cand) as fh:
            d = json.load(fh)
        return {"hbm_gbs": float(d["hbm_gbs"]), "bf16_tflops_sustained": float(d.get("bf16_tflops_sustained", d.get("bf16_tflops"))),
                "source": os.path.basename(cand)}
    return dict(NOMINAL)


def muon_shapes(cfg: ModelConfig) -> list[tuple[int, int, int]]:
    """(rows, cols, count) of the matrices Muon orthogonalises."""
    d, f, L = cfg.hidden_size, cfg.intermediate_size, cfg.num_layers
    return [(cfg.q_dim, d, L), (cfg.kv_dim, d, 2 * L), (d, cfg.q_dim, L), (f, d, 2 * L), (d, f, L)]


def train_ops(cfg: ModelConfig, tokens: int, seq: int, dp: int, tp: int, ns_iters: int = 5) -> list[dict[str, Any]]:
    """Per-GPU work of one optimizer step with one micro-batch of ``tokens`` tokens (before the TP division)."""
    d, f, L, V = cfg.hidden_size, cfg.intermediate_size, cfg.num_layers, cfg.vocab_size
    n = tokens
    ops: list[dict[str, Any]] = []

    def add(name: str, flops: float = 0.0, nbytes: float = 0.0) -> None:
        ops.append({"op": name, "flops": flops, "bytes": nbytes})
    proj = cfg.matmul_params() - V * d
    add("projections (fwd, dgrad, wgrad)", 6.0 * proj * n / tp)
    add("loss head products", 6.0 * V * d * n / tp)
    # causal attention: forward QK^T and PV (2 x 2 x T/2 x q_dim per token), backward five products
    add("attention forward", 2 * 2 * L * cfg.q_dim * (seq / 2) * n / tp)
    add("attention backward", 5 * 2 * L * cfg.q_dim * (seq / 2) * n / tp)
    ns = 0.0
    for r, c, cnt in muon_shapes(cfg):
        m, k = min(r, c), max(r, c)
        ns += cnt * ns_iters * (m * m * k + m ** 3 + 2.0 * m * m * k)
    add("Newton-Schulz", ns / (dp * tp))
    act = 2.0 * n * d / tp                          # one bf16 token-major tensor (token-sharded under sequence parallelism)
    if cfg.attn_res:
        bounds = sorted(cfg.boundaries())
        committed_reads = sum(range(1, len(bounds) + 1))         # block b reads its b committed sources once
        calls = 2 * L + 1
        # forward: sources once per block; per call: partial in, normalised out.  backward: the same tensors again plus
        # the source gradients (read-modify-write) and the incoming gradient
        add("AttnRes routing forward", nbytes=act * (committed_reads + 2 * calls))
        add("AttnRes routing backward", nbytes=act * (3 * committed_reads + 4 * calls))
    else:
        add("RMSNorm forward + backward", nbytes=act * (2 + 4) * (2 * L + 1))
    qkv = 2.0 * n * (cfg.q_dim + 2 * cfg.kv_dim) / tp
    add("QK-norm + RoPE", nbytes=2 * qkv * 2)                    # read + write, forward and backward
    add("SwiGLU", nbytes=2.0 * n * f / tp * L * (3 + 5))         # fwd: gate, up in, h out; bwd: gate, up, dh in, dgate, dup out
    add("loss head logits traffic", nbytes=2.0 * n * V / tp * 4)
    params = cfg.param_count()
    muon_elems = sum(r * c * cnt for r, c, cnt in muon_shapes(cfg))
    adamw_elems = params - muon_elems
    # Muon: gradient + momentum read, momentum write, parameter read + write (bf16 grads / params, fp32 momentum)
    add("Muon momentum + apply", nbytes=muon_elems / (dp * tp) * (2 + 4 + 4 + 2 + 2))
    add("AdamW", nbytes=adamw_elems / tp * (2 + 4 * 4 + 2 + 2))
    return ops


def comm_floor_ms(cfg: ModelConfig, tokens: int, dp: int, tp: int) -> dict[str, float]:
    out: dict[str, float] = {}
    if dp > 1:
        grad_bytes = 2.0 * cfg.param_count() / tp
        out["dp gradient reduction + parameter publish"] = 2 * grad_bytes * (dp - 1) / dp / (NVLINK_GBS * 1e9) * 1e3
    if tp > 1:
        per = 2.0 * tokens * cfg.hidden_size * (tp - 1) / tp       # one gather or scatter of the token-major activation
        out["tp gathers and scatters"] = 4 * 2 * cfg.num_layers * per / (NVLINK_GBS * 1e9) * 1e3
    return out


def decode_bytes(cfg: ModelConfig, batch: int, context: float, tp: int) -> dict[str, float]:
    weights = 2.0 * cfg.matmul_params() / tp           # every projection and the vocabulary product; the embedding gather reads B rows
    kv = 2.0 * batch * context * cfg.num_layers * 2 * cfg.kv_dim / tp
    return {"weights": weights, "kv cache": kv}


def report(rows: list[dict[str, Any]], peaks: dict[str, Any]) -> float:
    total = 0.0
    for r in rows:
        r["ms"] = max(r["flops"] / (peaks["bf16_tflops_sustained"] * 1e12), r["bytes"] / (peaks["hbm_gbs"] * 1e9)) * 1e3
        total += r["ms"]
    return total


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("mode", choices=["train", "decode"])
    ap.add_argument("--model", default="3b", choices=sorted(MODEL_PRESETS))
    ap.add_argument("--no_attn_res", action="store_true")
    ap.add_argument("--blocks", type=int, default=7)
    ap.add_argument("--micro_batch", type=int, default=8)
    ap.add_argument("--seq", type=int, default=4096)
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--tp", type=int, default=1)
    ap.add_argument("--ns_iter", type=int, default=5)
    ap.add_argument("--batch", type=int, default=64, help="decode: requests in the batch")
    ap.add_argument("--context", type=float, default=1220.0, help="decode: mean cached tokens per request")
    ap.add_argument("--measured_ms", type=float, default=None)
    ap.add_argument("--peaks", default=None)
    ap.add_argument("--json", action="store_true")
    a = ap.parse_args()
    if a.mode == "train" and a.gpus % a.tp:
        raise SystemExit("--gpus must be a multiple of --tp")
    cfg = ModelConfig(**MODEL_PRESETS[a.model], attn_res=not a.no_attn_res, attn_res_n_blocks=min(a.blocks, MODEL_PRESETS[a.model]["num_layers"]))
    peaks = load_peaks(a.peaks)
    out: dict[str, Any] = {"mode": a.mode, "model": a.model, "peaks": peaks}
    if a.mode == "train":
        dp = a.gpus // a.tp
        tokens = a.micro_batch * a.seq                 # per data-parallel rank; a TP group shares them
        rows = train_ops(cfg, tokens, a.seq, dp, a.tp, a.ns_iter)
        floor = report(rows, peaks)
        comm = comm_floor_ms(cfg, tokens, dp, a.tp)
        out.update(tokens_per_step=tokens * dp, ops=rows, floor_ms=floor, comm_floor_ms=comm,
                   compute_only_floor_ms=sum(r["flops"] for r in rows if r["op"] != "Newton-Schulz")
                   / (peaks["bf16_tflops_sustained"] * 1e12) * 1e3)
    else:
        b = decode_bytes(cfg, a.batch, a.context, a.tp)
        rows = [{"op": k, "flops": 0.0, "bytes": v} for k, v in b.items()]
        floor = report(rows, peaks)
        out.update(ops=rows, floor_ms=floor, tokens_per_s_at_floor=a.batch / (floor / 1e3))
    if a.measured_ms:
        out["measured_ms"] = a.measured_ms
        out["fraction_of_floor"] = out["floor_ms"] / a.measured_ms
    if a.json:
        print(json.dumps(out))
        return
    print(f"{a.mode} floor for {a.model} ({'AttnRes, ' + str(cfg.attn_res_n_blocks) + ' blocks' if cfg.attn_res else 'no AttnRes'}); "
          f"peaks from {peaks['source']}: {peaks['hbm_gbs']:.0f} GB/s, {peaks['bf16_tflops_sustained']:.0f} TFLOP/s")
    print(f"{'op':<42}{'GFLOP':>12}{'GB':>10}{'floor ms':>10}")
    for r in rows:
        print(f"{r['op']:<42}{r['flops'] / 1e9:>12.0f}{r['bytes'] / 1e9:>10.2f}{r['ms']:>10.3f}")
    print(f"{'sum of the per-op floors':<42}{'':>22}{out['floor_ms']:>10.3f}")
    if a.mode == "train":
        print(f"{'products and attention alone':<42}{'':>22}{out['compute_only_floor_ms']:>10.3f}")
        for k, v in out["comm_floor_ms"].items():
            print(f"{'NVLink: ' + k:<64}{v:>10.3f}")
    else:
        print(f"tokens/s at the floor: {out['tokens_per_s_at_floor']:.0f}")
    if a.measured_ms:
        print(f"measured {a.measured_ms:.2f} ms: {out['fraction_of_floor']:.2f} of the floor")


if __name__ == "__main__":
    main()
