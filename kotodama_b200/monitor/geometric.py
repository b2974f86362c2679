"""Geometric health monitoring of a training run (rank 0, on a fixed probe batch).

Tier 1 (cheap, every few hundred steps): RankMe of the last layer's hidden states (entropy of
the normalised singular values), stable rank ``||W||_F^2 / ||W||_2^2`` of sampled projection
matrices, dead-unit fraction, anisotropy (mean pairwise cosine), attention-entropy statistics,
and for AttnRes the final aggregation's mean depth weights and block norms.
Tier 2 (every few thousand steps): power-law exponent of each matrix's spectrum (log-log fit,
the WeightWatcher-style proxy) and the TwoNN intrinsic dimension of hidden states.

Metric names follow the reference (``src/monitoring/geometric.py:185-230,266-293,352,511-513``):
``geo/rankme_last``, ``geo/layer_{i}/stable_rank_{proj}``, ``geo/layer_{i}/dead_units``,
``geo/layer_{i}/anisotropy``, ``geo/layer_{i}/attn_entropy_{mean,std}``, ``geo/ww_alpha_*``,
``geo/twonn_id/layer_{i}``, ``attnres/final_alpha/block_{b}``, ``attnres/block_norm/{b}``.
The probe forward walks the model's own modules, including the commit-and-reset of the partial
sum at block boundaries.
"""
from __future__ import annotations

import logging
import math
import time
from dataclasses import dataclass, field
from typing import Any, Optional

import torch

from ..models.llama import route_sources

logger = logging.getLogger(__name__)


@dataclass
class MonitorConfig:
    tier1_every: int = 500
    tier1_probe_size: int = 1024
    tier1_sample_layers: list[int] = field(default_factory=list)     # empty: 0, L/4, L/2, 3L/4, last
    tier2_every: int = 5000
    tier2_twonn_samples: int = 3000
    tier2_twonn_layers: list[int] = field(default_factory=list)      # empty: five evenly spaced
    tier3_token_checkpoints: list[int] = field(
        default_factory=lambda: [0, 8_000_000_000, 24_000_000_000, 48_000_000_000, 80_000_000_000])
    device: str = "cuda"
    max_probe_tokens: int = 16384


# ----------------------------------------------------------------------------- metrics
def rankme(H: torch.Tensor, eps: float = 1e-7) -> float:
    try:
        s = torch.linalg.svdvals(H.float())
        s = s / (s.sum() + eps)
        s = s[s > eps]
        return float(torch.exp(-(s * s.log()).sum()))
    except Exception:       # noqa: BLE001 - SVD may fail on degenerate input
        return 0.0


def stable_rank(W: torch.Tensor) -> float:
    try:
        w = W.float()
        return float(w.pow(2).sum() / (torch.linalg.svdvals(w)[0].pow(2) + 1e-10))
    except Exception:       # noqa: BLE001
        return 0.0


def dead_unit_fraction(hidden: torch.Tensor, threshold: float = 1e-6) -> float:
    return float((hidden.float().abs().mean(dim=tuple(range(hidden.ndim - 1))) < threshold).float().mean())


def anisotropy(H: torch.Tensor, max_samples: int = 512) -> float:
    if H.shape[0] > max_samples:
        H = H[torch.randperm(H.shape[0], device=H.device)[:max_samples]]
    Hn = torch.nn.functional.normalize(H.float(), dim=-1)
    n = Hn.shape[0]
    if n < 2:
        return 0.0
    sim = Hn @ Hn.t()
    return float((sim.sum() - sim.diagonal().sum()) / (n * (n - 1)))


def attention_entropy_stats(attn: torch.Tensor, eps: float = 1e-10) -> tuple[float, float]:
    a = attn.float().clamp(min=eps)
    per_head = (-(a * a.log()).sum(-1)).mean(dim=(0, 2))
    return float(per_head.mean()), float(per_head.std()) if per_head.numel() > 1 else 0.0


def _slope(x: torch.Tensor, y: torch.Tensor) -> float:
    xm, ym = x.mean(), y.mean()
    return float(((x - xm) * (y - ym)).sum() / ((x - xm).pow(2).sum() + 1e-10))


def spectrum_alpha(W: torch.Tensor, min_sv: int = 10) -> Optional[float]:
    """Negative log-log slope of the eigenvalues of ``W^T W`` against rank."""
    try:
        e = torch.linalg.svdvals(W.float().detach()).pow(2).sort(descending=True).values
        e = e[e > e[0] * 1e-10]
        if e.numel() < min_sv:
            return None
        alpha = -_slope(torch.log(torch.arange(1, e.numel() + 1, dtype=torch.float32, device=e.device)), e.log())
        return alpha if 0.1 <= alpha <= 20 else None
    except Exception:       # noqa: BLE001
        return None


def twonn_id(X: torch.Tensor, max_points: int = 5000) -> Optional[float]:
    """TwoNN intrinsic dimension (Facco et al. 2017): slope of ``log(1-F(mu))`` against ``log mu``
    with ``mu = r2/r1`` the ratio of second to first neighbour distance."""
    try:
        X = X.float()[:max_points]
        if X.shape[0] < 10:
            return None
        d = torch.cdist(X, X)
        d.fill_diagonal_(float("inf"))
        r = d.topk(2, dim=1, largest=False).values
        ok = r[:, 0] > 1e-10
        if int(ok.sum()) < 10:
            return None
        mu = (r[ok, 1] / r[ok, 0]).sort().values
        n = mu.numel()
        i = torch.arange(1, n + 1, dtype=torch.float32, device=X.device)
        dim = -_slope(mu.log(), torch.log(1.0 - i / (n + 1)))
        return dim if 0.5 <= dim <= 10000 else None
    except Exception:       # noqa: BLE001
        return None


def _std(v: list[float]) -> float:
    if len(v) < 2:
        return 0.0
    m = sum(v) / len(v)
    return (sum((x - m) ** 2 for x in v) / (len(v) - 1)) ** 0.5


# ----------------------------------------------------------------------------- monitor
class GeometricMonitor:
    def __init__(self, model: Any, config: Optional[MonitorConfig] = None) -> None:
        self.model = model.module if hasattr(model, "module") else model
        self.config = config or MonitorConfig()
        L = len(self.model.layers)
        # default layer samples as in the reference (``src/monitoring/geometric.py:108-124``): the metric keys carry the
        # layer index, so runs monitored by either code base line up
        if not self.config.tier1_sample_layers:
            step = max(1, L // 4)
            self.config.tier1_sample_layers = sorted({0, step, 2 * step, 3 * step, L - 1})
        if not self.config.tier2_twonn_layers:
            self.config.tier2_twonn_layers = [0, L // 4, L // 2, 3 * L // 4, L - 1]
        self._probe: Optional[torch.Tensor] = None
        self._attnres: dict[str, float] = {}

    def set_probe_batch(self, input_ids: torch.Tensor) -> None:
        self._probe = input_ids.clone()
        logger.info("Probe batch set: shape %s", tuple(input_ids.shape))

    # ---- probe forward -------------------------------------------------------
    @torch.no_grad()
    def _probe_forward(self, ids: torch.Tensor, want_attn: set[int]) -> tuple[dict[int, torch.Tensor], dict[int, torch.Tensor]]:
        """One state per layer and the attention probabilities of ``want_attn`` (first four sequences).
        Without AttnRes the state is the residual stream after the layer; with AttnRes it is the routed
        state the layer's attention reads, and for the last layer the final aggregation (before the
        output norm) - the captures of the reference's monitor, so that both produce the same series.
        The attention probabilities are always those the layer really used (the reference's plain path
        feeds the layer's output back into the same layer's attention instead)."""
        m = self.model
        cfg = m.config
        x = m.embed_tokens(ids)
        hidden: dict[int, torch.Tensor] = {}
        attn: dict[int, torch.Tensor] = {}
        T = ids.shape[1]
        causal = torch.ones(T, T, dtype=torch.bool, device=ids.device).tril()

        def attention(layer, h, idx):
            q, k, v = layer.attn.project_qkv(h, m.rope_cos, m.rope_sin)
            g = q.shape[1] // k.shape[1]
            k2, v2 = k.repeat_interleave(g, 1), v.repeat_interleave(g, 1)
            sc = (q.float() @ k2.float().transpose(-1, -2)) / math.sqrt(q.shape[-1])
            p = torch.softmax(sc.masked_fill(~causal, float("-inf")), -1)
            if idx in want_attn:
                attn[idx] = p[:4]                    # the first sequences only, as the reference does, to bound memory
            o = (p @ v2.float()).to(h.dtype).transpose(1, 2).reshape(h.shape[0], T, -1)
            return layer.attn.o_proj(o)

        if not cfg.attn_res:
            for i, layer in enumerate(m.layers):
                x = x + attention(layer, layer.attn_norm(x), i)
                x = x + layer.ffn(layer.ffn_norm(x))
                hidden[i] = x
            return hidden, attn
        committed: list[torch.Tensor] = []
        partial: Optional[torch.Tensor] = x
        bset = m._attn_res_boundary_set
        for i, layer in enumerate(m.layers):
            h = route_sources(committed + [partial], layer.attn_res_query, layer.attn_res_norm.weight,
                              layer.attn_res_norm.eps)
            if i in bset:
                committed.append(partial)
                partial = None                       # the new block starts from zero
            hidden[i] = h                            # the routed state the attention sub-layer reads (``geometric.py:463-476`` there)
            a = attention(layer, layer.attn_norm(h), i)
            partial = a if partial is None else partial + a
            h2 = route_sources(committed + [partial], layer.mlp_res_query, layer.mlp_res_norm.weight,
                               layer.mlp_res_norm.eps)
            partial = partial + layer.ffn(layer.ffn_norm(h2))
        srcs = committed + [partial]
        w = (m.final_res_query * m.final_res_norm.weight).float()
        u = torch.stack(srcs, 0).float()
        r = torch.rsqrt(u.pow(2).mean(-1) + m.final_res_norm.eps)
        alpha = torch.softmax((u * w).sum(-1) * r, 0).mean(dim=(1, 2))
        self._attnres = {}
        for b in range(len(srcs)):
            self._attnres[f"attnres/final_alpha/block_{b}"] = float(alpha[b])
            self._attnres[f"attnres/block_norm/{b}"] = float(u[b].norm(dim=-1).mean())
        # the last entry is the final aggregation itself (before the output norm), as in the reference's monitor
        hidden[len(m.layers) - 1] = (torch.softmax((u * w).sum(-1) * r, 0).unsqueeze(-1) * u).sum(0).to(x.dtype)
        return hidden, attn

    def _batch(self, probe: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
        b = probe if probe is not None else self._probe
        if b is None:
            return None
        dev = next(self.model.parameters()).device
        rows = max(1, min(b.shape[0], self.config.max_probe_tokens // max(b.shape[1], 1)))
        return b[:rows].to(dev)

    # ---- tiers ---------------------------------------------------------------------
    @torch.no_grad()
    def tier1(self, step: int, probe_batch: Optional[torch.Tensor] = None) -> dict[str, float]:
        t0 = time.time()
        batch = self._batch(probe_batch)
        if batch is None:
            logger.warning("No probe batch set: skipping Tier 1 metrics")
            return {}
        layers = set(self.config.tier1_sample_layers)
        hidden, attn = self._probe_forward(batch, layers)
        L = len(self.model.layers)
        out: dict[str, float] = {"geo/rankme_last": rankme(hidden[L - 1].reshape(-1, hidden[L - 1].shape[-1]))}
        for i in sorted(layers):
            layer, pre = self.model.layers[i], f"geo/layer_{i}"
            for name, w in (("q_proj", layer.attn.q_proj.weight), ("k_proj", layer.attn.k_proj.weight),
                            ("o_proj", layer.attn.o_proj.weight), ("gate_proj", layer.ffn.gate_proj.weight),
                            ("down_proj", layer.ffn.down_proj.weight)):
                out[f"{pre}/stable_rank_{name}"] = stable_rank(w)
            if i in hidden:
                out[f"{pre}/dead_units"] = dead_unit_fraction(hidden[i])
                out[f"{pre}/anisotropy"] = anisotropy(hidden[i].reshape(-1, hidden[i].shape[-1]))
            if i in attn:
                out[f"{pre}/attn_entropy_mean"], out[f"{pre}/attn_entropy_std"] = attention_entropy_stats(attn[i])
        out.update(self._attnres)
        out["geo/tier1_time_s"] = time.time() - t0
        out["geo/step"] = float(step)
        logger.info("Tier 1 geo: step=%d RankMe=%.1f (%.2fs)", step, out["geo/rankme_last"], out["geo/tier1_time_s"])
        return out

    @torch.no_grad()
    def tier2(self, step: int, probe_batch: Optional[torch.Tensor] = None) -> dict[str, float]:
        t0 = time.time()
        out: dict[str, float] = {}
        alphas: list[float] = []
        by_type: dict[str, list[float]] = {}
        for i, layer in enumerate(self.model.layers):
            for name, w in (("q_proj", layer.attn.q_proj.weight), ("k_proj", layer.attn.k_proj.weight),
                            ("v_proj", layer.attn.v_proj.weight), ("o_proj", layer.attn.o_proj.weight),
                            ("gate_proj", layer.ffn.gate_proj.weight), ("up_proj", layer.ffn.up_proj.weight),
                            ("down_proj", layer.ffn.down_proj.weight)):
                a = spectrum_alpha(w)
                if a is not None:
                    alphas.append(a)
                    by_type.setdefault(name, []).append(a)
                    out[f"geo/ww_alpha/layer_{i}/{name}"] = a
        if alphas:
            out["geo/ww_alpha_mean"] = sum(alphas) / len(alphas)
            out["geo/ww_alpha_std"] = _std(alphas)
            out["geo/ww_alpha_min"], out["geo/ww_alpha_max"] = min(alphas), max(alphas)
            out["geo/ww_alpha_healthy_frac"] = sum(2.0 < a < 4.0 for a in alphas) / len(alphas)      # the reference's band
            for k, v in by_type.items():
                out[f"geo/ww_alpha_by_type/{k}"] = sum(v) / len(v)
        batch = self._batch(probe_batch)
        if batch is not None:
            hidden, _ = self._probe_forward(batch, set())
            for i in self.config.tier2_twonn_layers:
                if i in hidden:
                    X = hidden[i].reshape(-1, hidden[i].shape[-1])[: self.config.tier2_twonn_samples]
                    d = twonn_id(X)
                    if d is not None:
                        out[f"geo/twonn_id/layer_{i}"] = d
        out["geo/tier2_time_s"] = time.time() - t0
        return out
