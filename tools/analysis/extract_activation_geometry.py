#!/usr/bin/env python
"""Activation-geometry extraction (track 5a): geometric objects of a checkpoint's residual stream,
attention and weights, written as arrays for the visualiser and as a JSON summary for the report.

Components (``--components``, comma separated, or ``all``):

  needs forward passes
    point_clouds       mean-pooled state of every sequence after every layer  -> point_clouds.npz
    topo_clouds        token-level states of a few layers, subsampled (2000 points per layer by
                       default) with a TwoNN intrinsic-dimension estimate      -> topo_clouds.npz
    trajectories       last-token state of every prompt through the layers     -> trajectories.npz
    eigenspectra       covariance spectrum of the token states per layer (participation ratio, RankMe)
    attention          attention matrices of selected layers per prompt        -> attention_weights.npz
                       (+ per-head entropy and mean attention distance of those layers)
    attention_outputs  mean-pooled attention-branch output per layer           -> attention_outputs.npz
    head_entropy       per-head attention entropy of EVERY layer over sequences -> head_entropy.npz
  weights only (no forward pass, CPU is enough)
    weight_spectra     singular values of q/k/v/o/gate/up/down per layer        -> weight_spectra.npz
    effective_rank     participation ratio, stable rank and entropy rank of those spectra
  across runs (after the per-run passes, or alone from files written earlier)
    procrustes         point clouds of all runs projected on their joint principal axes per layer
                       (-> _pairs/procrustes.npz) and the orthogonal-Procrustes distance per layer pair

Sequences come from ``--eval-data`` (a flat uint16 token file, ``--n-seqs`` rows of ``--seq-len``) or, without
it, from the prompt set (one sequence per prompt).

    python tools/analysis/extract_activation_geometry.py --checkpoint ckpt.pt --name run --device cuda
    python tools/analysis/extract_activation_geometry.py --checkpoints a,b --components point_clouds,procrustes \\
        --eval-data data/eval.bin --n-seqs 500 --seq-len 512
    python tools/analysis/extract_activation_geometry.py --checkpoint ckpt.pt --components weight_spectra,effective_rank
    python tools/analysis/extract_activation_geometry.py --components procrustes --runs a,b      # from files written earlier

Writes ``<output-dir>/<run>/activation_geometry/{geometry.json, arrays.npz, <component>.npz}``.  Counterpart of the
reference's ``scripts/analysis/extract_activation_geometry.py`` (same components; one directory per run instead of
run-prefixed keys in shared files).
"""
from __future__ import annotations

import argparse
import math
import time
from pathlib import Path
from typing import Any, Iterator

import numpy as np
import torch
from _common import ROOT, add_checkpoint_args, load_yaml, open_model, run_dir, select_checkpoints, tokenizer, write_json

from kotodama_b200.eval import forward_with_states

FORWARD = ["point_clouds", "topo_clouds", "trajectories", "eigenspectra", "attention", "attention_outputs", "head_entropy"]
WEIGHTS = ["weight_spectra", "effective_rank"]
ACROSS = ["procrustes"]
ALL = FORWARD + WEIGHTS + ACROSS
WEIGHT_TYPES = ["q_proj", "k_proj", "v_proj", "o_proj", "gate_proj", "up_proj", "down_proj"]


# ------------------------------------------------------------------------------ small numerics
def spectrum_stats(x: np.ndarray) -> dict:
    """Covariance spectrum of the rows of ``x``: participation ratio, RankMe (exp of the spectral entropy)."""
    x = x - x.mean(0, keepdims=True)
    s = np.linalg.svd(x, compute_uv=False) ** 2
    p = s / max(s.sum(), 1e-12)
    return {"participation_ratio": float(s.sum() ** 2 / max((s ** 2).sum(), 1e-12)),
            "rankme": float(math.exp(-(p * np.log(p + 1e-12)).sum())), "top": s[:16].tolist()}


def pca3(x: np.ndarray) -> np.ndarray:
    x = x - x.mean(0, keepdims=True)
    _, _, vt = np.linalg.svd(x, full_matrices=False)
    k = min(3, vt.shape[0])
    out = np.zeros((x.shape[0], 3), dtype=np.float32)
    out[:, :k] = x @ vt[:k].T
    return out


def twonn_dimension(x: np.ndarray, discard: float = 0.1) -> float:
    """TwoNN intrinsic dimension (Facco et al. 2017): the ratio of second to first neighbour distance of a
    point follows a Pareto law whose exponent is the dimension; fitted on all but the largest ``discard``."""
    n = len(x)
    if n < 8:
        return float("nan")
    sq = (x ** 2).sum(1)
    mu = np.empty(n)
    for lo in range(0, n, 512):                          # blocks keep the distance matrix small
        d2 = sq[lo:lo + 512, None] + sq[None, :] - 2.0 * x[lo:lo + 512] @ x.T
        d2[np.arange(d2.shape[0]), np.arange(lo, lo + d2.shape[0])] = np.inf
        part = np.partition(d2, 1, axis=1)[:, :2]
        r1, r2 = np.sqrt(np.maximum(part.min(1), 1e-24)), np.sqrt(np.maximum(part.max(1), 1e-24))
        mu[lo:lo + 512] = r2 / r1
    mu = np.sort(mu[np.isfinite(mu) & (mu > 1.0)])
    keep = mu[: max(4, int(len(mu) * (1.0 - discard)))]
    if len(keep) < 4:
        return float("nan")
    # F(mu) = 1 - mu^-d  =>  -log(1 - F) = d log(mu): least squares through the origin
    lx = np.log(keep)
    ly = -np.log1p(-np.minimum(np.arange(1, len(keep) + 1) / len(mu), 1 - 1e-9))
    return float((lx @ ly) / max(lx @ lx, 1e-300))


def rank_stats(sv: np.ndarray) -> dict:
    s = sv.astype(np.float64)
    q = s / max(s.sum(), 1e-300)
    return {"participation_ratio": float(s.sum() ** 2 / max((s ** 2).sum(), 1e-300)),
            "stable_rank": float((s ** 2).sum() / max(s[0] ** 2, 1e-300)),
            "entropy_rank": float(math.exp(-(q * np.log(q + 1e-300)).sum()))}


def procrustes_distance(a: np.ndarray, b: np.ndarray) -> float:
    a = (a - a.mean(0)) / (np.linalg.norm(a - a.mean(0)) + 1e-12)
    b = (b - b.mean(0)) / (np.linalg.norm(b - b.mean(0)) + 1e-12)
    s = np.linalg.svd(a.T @ b, compute_uv=False)
    return float(max(0.0, 1.0 - s.sum() ** 2))


# ------------------------------------------------------------------------------ sequences
def eval_batches(path: str, n_seqs: int, seq_len: int, batch: int, vocab: int, device: str) -> Iterator[torch.Tensor]:
    """``n_seqs`` rows of ``seq_len`` tokens from a flat little-endian uint16 file, ``batch`` rows at a time."""
    data = np.memmap(path, dtype="<u2", mode="r")
    n = min(n_seqs, len(data) // seq_len)
    if n == 0:
        raise SystemExit(f"{path}: fewer than {seq_len} tokens")
    for lo in range(0, n, batch):
        rows = np.stack([np.asarray(data[(lo + j) * seq_len:(lo + j + 1) * seq_len]) for j in range(min(batch, n - lo))])
        yield torch.from_numpy(rows.astype(np.int64) % vocab).to(device)


def prompt_batches(tok: Any, prompts: list[str], max_len: int, device: str) -> Iterator[torch.Tensor]:
    for p in prompts:
        yield torch.tensor([tok.encode(p)[:max_len]], device=device)


class Collector:
    """Accumulates what the forward-pass components need, batch by batch, so that one pass over the
    sequences serves all of them."""

    def __init__(self, model: Any, comps: set[str], topo_layers: list[int], attn_layers: list[int], topo_subsample: int,
                 keep_attention: int) -> None:
        self.L = model.config.num_layers
        self.H = model.config.num_attention_heads
        self.comps = comps
        self.topo_layers, self.attn_layers = topo_layers, attn_layers
        self.topo_subsample, self.keep_attention = topo_subsample, keep_attention
        self.pooled: list[list[np.ndarray]] = [[] for _ in range(self.L + 1)]          # mean over tokens, per layer
        self.last: list[np.ndarray] = []                                               # [L+1, D] per sequence
        self.tokens: dict[int, list[np.ndarray]] = {l: [] for l in topo_layers}
        self.cov_rows: list[list[np.ndarray]] = [[] for _ in range(self.L + 1)]
        self.branch: list[list[np.ndarray]] = [[] for _ in range(self.L)]
        self.branch_ratio = np.zeros(self.L)
        self.entropy = np.zeros((self.L, self.H))
        self.distance = np.zeros((self.L, self.H))
        self.positions = 0
        self.attn_saved: dict[str, np.ndarray] = {}
        self.n_seq = 0
        self._rng = np.random.RandomState(42)

    def _attention(self, layer: int, w: torch.Tensor) -> None:
        B, H, T, _ = w.shape
        ent = -(w * torch.log(w + 1e-10)).sum(-1)                                       # [B, H, T]
        idx = torch.arange(T, device=w.device, dtype=w.dtype)
        dist = (w * (idx[:, None] - idx[None, :]).abs()).sum(-1)
        self.entropy[layer] += ent.sum((0, 2)).double().cpu().numpy()
        self.distance[layer] += dist.sum((0, 2)).double().cpu().numpy()
        if "attention" in self.comps and layer in self.attn_layers:
            for b in range(B):
                if self.n_seq + b < self.keep_attention:
                    self.attn_saved[f"prompt_{self.n_seq + b}_layer_{layer}"] = w[b].float().cpu().numpy().astype(np.float16)

    def add(self, model: Any, ids: torch.Tensor) -> None:
        c = self.comps
        layers = list(range(self.L)) if "head_entropy" in c else (self.attn_layers if "attention" in c else [])
        res = forward_with_states(model, ids, attention_layers=layers, attention_fn=self._attention if layers else None,
                                  capture_attention_outputs="attention_outputs" in c)
        B, T = ids.shape
        for l, s in enumerate(res.states):
            sf = s.float()
            if c & {"point_clouds", "procrustes"}:
                self.pooled[l].append(sf.mean(1).cpu().numpy())
            if "eigenspectra" in c:
                flat = sf.reshape(B * T, -1)
                take = min(len(flat), 256)                                              # rows per batch that enter the spectrum
                sel = torch.from_numpy(self._rng.choice(len(flat), take, replace=False)).to(flat.device)
                self.cov_rows[l].append(flat[sel].cpu().numpy())
            if "topo_clouds" in c and l - 1 in self.tokens:
                self.tokens[l - 1].append(sf.reshape(B * T, -1).cpu().numpy())
        if "trajectories" in c:
            stack = torch.stack([s[:, -1].float() for s in res.states], 1).cpu().numpy()  # [B, L+1, D]
            self.last.extend(stack)
        if "attention_outputs" in c:
            for l, a in enumerate(res.attention_outputs):
                af = a.float()
                self.branch[l].append(af.mean(1).cpu().numpy())
                self.branch_ratio[l] += float((af.norm(dim=-1) / (res.states[l + 1].float().norm(dim=-1) + 1e-9)).sum())
        self.positions += B * T
        self.n_seq += B

    # ---- what the accumulated pieces turn into: (summary for geometry.json, {file name: arrays})
    def finish(self) -> tuple[dict, dict[str, dict[str, np.ndarray]], dict[str, np.ndarray]]:
        c, L = self.comps, self.L
        out: dict[str, Any] = {"sequences": self.n_seq, "positions": self.positions}
        files: dict[str, dict[str, np.ndarray]] = {}
        arrays: dict[str, np.ndarray] = {}
        if c & {"point_clouds", "procrustes"} and self.pooled[0]:
            clouds = [np.concatenate(p) for p in self.pooled]                           # [n_seq, D] per layer
            files["point_clouds"] = {f"layer_{l - 1}": x.astype(np.float32) for l, x in enumerate(clouds)}   # -1 = embeddings
            if "point_clouds" in c:
                arrays["point_clouds"] = np.stack([pca3(x) for x in clouds])            # [L+1, n_seq, 3] for the plots
                out["point_clouds"] = {"spread_per_layer": [float(np.linalg.norm(x - x.mean(0), axis=1).mean()) for x in clouds]}
        if "topo_clouds" in c:
            topo, dims = {}, {}
            for l, parts in self.tokens.items():
                full = np.concatenate(parts)
                sel = self._rng.choice(len(full), min(self.topo_subsample, len(full)), replace=False)
                topo[f"layer_{l}"] = full[sel].astype(np.float32)
                dims[str(l)] = twonn_dimension(full[sel].astype(np.float64))
            files["topo_clouds"] = topo
            out["topo_clouds"] = {"points_per_layer": {k: int(len(v)) for k, v in topo.items()}, "twonn_dimension": dims}
        if "eigenspectra" in c:
            out["eigenspectra"] = [spectrum_stats(np.concatenate(r)) for r in self.cov_rows]
        if "trajectories" in c and self.last:
            last = np.stack(self.last)                                                   # [n_seq, L+1, D]
            norms = np.linalg.norm(last, axis=-1)
            d = np.diff(last, axis=1)
            step = np.linalg.norm(d, axis=-1)
            cos = (d[:, 1:] * d[:, :-1]).sum(-1) / (step[:, 1:] * step[:, :-1] + 1e-9)
            net = np.linalg.norm(last[:, -1] - last[:, 0], axis=-1)
            out["trajectories"] = {"mean_norm_per_layer": norms.mean(0).tolist(), "mean_step_cosine": cos.mean(0).tolist(),
                                   "mean_step_length": step.mean(0).tolist(),
                                   "straightness": float((net / (step.sum(1) + 1e-9)).mean())}   # 1 = a straight line through depth
            arrays["trajectory_norms"] = norms
            files["trajectories"] = {f"prompt_{j}": t.astype(np.float32) for j, t in enumerate(last)}
        if c & {"attention", "head_entropy"} and self.positions:
            ent, dist = self.entropy / self.positions, self.distance / self.positions
            if "head_entropy" in c:
                files["head_entropy"] = {"entropy": ent.astype(np.float32), "mean_distance": dist.astype(np.float32)}
                out["head_entropy"] = {"mean_per_layer": ent.mean(1).tolist(), "min_per_layer": ent.min(1).tolist(),
                                       "most_focused_head": [int(x) for x in ent.argmin(1)]}
            if "attention" in c:
                out["attention"] = {str(l): {"head_entropy": ent[l].tolist(), "mean_attention_distance": dist[l].tolist()}
                                    for l in self.attn_layers}
                if self.attn_saved:
                    files["attention_weights"] = self.attn_saved
        if "attention_outputs" in c and self.branch[0]:
            files["attention_outputs"] = {f"layer_{l}": np.concatenate(b).astype(np.float32) for l, b in enumerate(self.branch)}
            out["attention_outputs"] = {"branch_to_state_norm_ratio": (self.branch_ratio / max(self.positions, 1)).tolist(),
                                        "spectrum": [spectrum_stats(np.concatenate(b)) for b in self.branch]}
        return out, files, arrays


# ------------------------------------------------------------------------------ weights
def weight_spectra(model: Any) -> dict[str, np.ndarray]:
    """Singular values of every projection: ``{"<type>_layer_<i>": sv}``."""
    out = {}
    for i, layer in enumerate(model.layers):
        mods = {"q_proj": layer.attn.q_proj, "k_proj": layer.attn.k_proj, "v_proj": layer.attn.v_proj, "o_proj": layer.attn.o_proj,
                "gate_proj": layer.ffn.gate_proj, "up_proj": layer.ffn.up_proj, "down_proj": layer.ffn.down_proj}
        for name, mod in mods.items():
            out[f"{name}_layer_{i}"] = torch.linalg.svdvals(mod.weight.detach().float().cpu()).numpy()
    return out


def effective_ranks(spectra: dict[str, np.ndarray], n_layers: int) -> dict[str, dict[str, list[float]]]:
    """Per weight type, one list over layers of each rank measure."""
    res: dict[str, dict[str, list[float]]] = {}
    for t in WEIGHT_TYPES:
        rows = [rank_stats(spectra[f"{t}_layer_{i}"]) if f"{t}_layer_{i}" in spectra else None for i in range(n_layers)]
        res[t] = {k: [r[k] if r else float("nan") for r in rows] for k in ("participation_ratio", "stable_rank", "entropy_rank")}
    return res


# ------------------------------------------------------------------------------ across runs
def joint_alignment(clouds: dict[str, dict[str, np.ndarray]], n_components: int) -> tuple[dict[str, np.ndarray], dict[str, list[float]]]:
    """Per layer: centre and scale every run's cloud, project all of them on the principal axes of their union
    (so that runs can be drawn in one frame), and measure the orthogonal-Procrustes distance of every pair."""
    runs = list(clouds)
    layers = sorted(set.intersection(*[set(c) for c in clouds.values()]), key=lambda k: int(k.split("_")[1]))
    aligned: dict[str, np.ndarray] = {}
    dist: dict[str, list[float]] = {f"{x}|{y}": [] for i, x in enumerate(runs) for y in runs[i + 1:]}
    for key in layers:
        normed = {}
        for r in runs:
            x = clouds[r][key].astype(np.float64)
            x = x - x.mean(0, keepdims=True)
            normed[r] = x / max(np.linalg.norm(x), 1e-12)
        if len({v.shape[1] for v in normed.values()}) == 1:                             # same width: one joint basis
            union = np.concatenate(list(normed.values()))
            _, _, vt = np.linalg.svd(union - union.mean(0, keepdims=True), full_matrices=False)
            top = vt[: min(n_components, len(vt))].T
            for r in runs:
                aligned[f"{r}_{key}"] = (normed[r] @ top).astype(np.float32)
        for i, x in enumerate(runs):
            for y in runs[i + 1:]:
                n = min(len(normed[x]), len(normed[y]))
                same = normed[x].shape[1] == normed[y].shape[1]
                dist[f"{x}|{y}"].append(procrustes_distance(normed[x][:n], normed[y][:n]) if same else float("nan"))
    return aligned, dist


# ------------------------------------------------------------------------------ driver
def parse_layers(spec: str, L: int) -> list[int]:
    return sorted({int(x) % L for x in spec.split(",") if x.strip()})


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_checkpoint_args(ap)
    ap.add_argument("--components", default="all")
    ap.add_argument("--prompt-set", default="extended")
    ap.add_argument("--prompts-file", default=str(ROOT / "configs" / "prompts.yaml"))
    ap.add_argument("--eval-data", default=None, help="flat uint16 token file; without it the prompt set supplies the sequences")
    ap.add_argument("--n-seqs", type=int, default=500)
    ap.add_argument("--seq-len", type=int, default=512)
    ap.add_argument("--batch-size", type=int, default=16)
    ap.add_argument("--attention-layers", default="0,-1", help="layers whose attention matrices are kept (negative: from the end)")
    ap.add_argument("--keep-attention", type=int, default=8, help="sequences whose attention matrices are saved")
    ap.add_argument("--topo-layers", default="0,-1", help="layers for the token-level clouds; the middle layer is added")
    ap.add_argument("--topo-subsample", type=int, default=2000)
    ap.add_argument("--procrustes-components", type=int, default=50)
    ap.add_argument("--runs", default=None,
                    help="with --components procrustes: names of runs already extracted into --output-dir (no model is loaded)")
    a = ap.parse_args()
    comps = set(ALL) if a.components == "all" else {c.strip() for c in a.components.split(",") if c.strip()}
    unknown = comps - set(ALL)
    if unknown:
        raise SystemExit(f"unknown components {sorted(unknown)}; choose from {ALL}")
    prompts = load_yaml(a.prompts_file)[a.prompt_set]
    tok = tokenizer(a.tokenizer) if comps & set(FORWARD + ACROSS) and not a.eval_data else None
    from_disk = comps == {"procrustes"} and a.runs
    selected = [(r.strip(), {}) for r in a.runs.split(",")] if from_disk else select_checkpoints(a)
    clouds_by_run: dict[str, dict[str, np.ndarray]] = {}
    for run, kw in selected:
        t0 = time.time()
        d = run_dir(a.output_dir, run, "activation_geometry")
        fwd = comps & set(FORWARD) or ("procrustes" in comps and not (d / "point_clouds.npz").exists())
        if from_disk or not (fwd or comps & set(WEIGHTS)):
            continue
        model, _ = open_model(kw, a.device)
        L = model.config.num_layers
        out: dict[str, Any] = {"run": run, "layers": L, "components": sorted(comps)}
        arrays: dict[str, np.ndarray] = {}
        if fwd:
            topo = sorted(set(parse_layers(a.topo_layers, L)) | {L // 2})
            col = Collector(model, comps, topo, parse_layers(a.attention_layers, L), a.topo_subsample, a.keep_attention)
            if a.eval_data:
                batches = eval_batches(a.eval_data, a.n_seqs, a.seq_len, a.batch_size, model.config.vocab_size, a.device)
                out["source"] = {"eval_data": a.eval_data, "seq_len": a.seq_len}
            else:
                batches = prompt_batches(tok, prompts, model.config.max_position_embeddings, a.device)
                out["source"] = {"prompt_set": a.prompt_set}
            for ids in batches:
                col.add(model, ids)
            summary, files, arrays = col.finish()
            out.update(summary)
            out["prompts"] = col.n_seq
            for name, content in files.items():
                np.savez_compressed(d / f"{name}.npz", **content)
            if "point_clouds" in files:
                clouds_by_run[run] = files["point_clouds"]
        if comps & set(WEIGHTS):
            sp = weight_spectra(model)
            if "weight_spectra" in comps:
                np.savez_compressed(d / "weight_spectra.npz", **sp)
                out["weight_spectra"] = {t: [float(sp[f"{t}_layer_{i}"][0]) for i in range(L)] for t in WEIGHT_TYPES}   # top singular value
            if "effective_rank" in comps:
                out["effective_rank"] = effective_ranks(sp, L)
        write_json(d / "geometry.json", out)
        if arrays:
            np.savez_compressed(d / "arrays.npz", **arrays)
        print(f"{run}: {sorted(comps - set(ACROSS))} -> {d} ({time.time() - t0:.1f}s)")
        del model
    if "procrustes" in comps:
        for run, _ in selected:                          # runs extracted earlier: read their clouds from disk
            f = Path(a.output_dir) / run / "activation_geometry" / "point_clouds.npz"
            if run not in clouds_by_run and f.exists():
                with np.load(f) as z:
                    clouds_by_run[run] = {k: z[k] for k in z.files}
        if len(clouds_by_run) < 2:
            print("procrustes: needs the point clouds of at least two runs (--checkpoints a,b)")
            return
        aligned, dist = joint_alignment(clouds_by_run, a.procrustes_components)
        pd = run_dir(a.output_dir, "_pairs")
        np.savez_compressed(pd / "procrustes.npz", run_names=np.array(list(clouds_by_run)), **aligned)
        write_json(pd / "procrustes.json", dist)
        print(f"procrustes: {len(dist)} pairs -> {pd}")


if __name__ == "__main__":
    main()
