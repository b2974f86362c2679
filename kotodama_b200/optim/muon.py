"""Muon (momentum orthogonalised by Newton-Schulz) + AdamW hybrid and the WSD schedule.

Behavioural parity with the reference ``src/training/muon.py``:

* coefficient presets ``original`` / ``gram_ns`` / ``polar_express`` (``muon.py:45-83``);
* Newton-Schulz in fp16 on the Nesterov update, tall matrices transposed, Frobenius
  normalisation with ``+1e-7`` (``muon.py:104-152``), same-shape matrices batched;
* update ``p *= 1 - lr*wd; p -= lr * max(1, sqrt(rows/cols)) * orth`` (``muon.py:349-351``);
* parameter split: 2-D and not embedding / LM head goes to Muon, the rest to AdamW
  (``muon.py:381``); ``ns_coefficients`` travels in the state dict (``muon.py:231-246``);
* warmup / stable / decay schedule with sqrt, linear or cosine decay (``muon.py:421-487``).

This file is the stand-alone ``torch.optim`` flavour (works with any autograd model on any
device).  The training executor runs the same math through flat arenas and fused kernels and
exchanges state with this class through the same state-dict layout.
"""
from __future__ import annotations

import logging
import math
from typing import Any, Optional

import torch
from torch.optim import AdamW, Optimizer

logger = logging.getLogger(__name__)

_SAFETY = 1.05
_PE_RAW = [
    (8.28721201814563, -23.595886519098837, 17.300387312530933),
    (4.107059111542203, -2.9478499167379106, 0.5448431082926601),
    (3.9486908534822946, -2.908902115962949, 0.5518191394370137),
    (3.3184196573706015, -2.488488024314874, 0.51004894012372),
    (2.300652019954817, -1.6689039845747493, 0.4188073119525673),
]
NS_COEFFICIENT_PRESETS: dict[str, list[tuple[float, float, float]]] = {
    "original": [(3.4445, -4.7750, 2.0315)] * 5,
    "gram_ns": [
        (4.0848, -6.8946, 2.9270),
        (3.9505, -6.3029, 2.6377),
        (3.7418, -5.5913, 2.3037),
        (2.8769, -3.1427, 1.2046),
        (2.8366, -3.0525, 1.2012),
    ],
    "polar_express": [(a / _SAFETY, b / _SAFETY ** 3, c / _SAFETY ** 5) for a, b, c in _PE_RAW],
}


def resolve_ns_coefficients(preset: Optional[str], num_iterations: int) -> list[tuple[float, float, float]]:
    """Per-iteration ``(a, b, c)``; the last entry repeats when more iterations are requested."""
    name = preset or "original"
    if name not in NS_COEFFICIENT_PRESETS:
        raise ValueError(f"Unknown NS coefficient preset '{name}'. Available: {list(NS_COEFFICIENT_PRESETS)}")
    table = NS_COEFFICIENT_PRESETS[name]
    return [table[min(i, len(table) - 1)] for i in range(num_iterations)]


def newton_schulz_orthogonalize(M: torch.Tensor, num_iterations: int = 5,
                                ns_coefficients: Optional[str] = None) -> torch.Tensor:
    """Approximate polar factor of ``M`` (2-D, or 3-D batch of same-shape matrices)."""
    assert M.ndim in (2, 3), f"Newton-Schulz needs a matrix or a batch of matrices, got {M.ndim}-D"
    X = M.half()
    tall = X.shape[-2] > X.shape[-1]
    if tall:
        X = X.transpose(-2, -1)
    X = X / (X.flatten(-2).norm(dim=-1)[..., None, None] + 1e-7)
    for a, b, c in resolve_ns_coefficients(ns_coefficients, num_iterations):
        A = X @ X.transpose(-2, -1)
        X = a * X + (b * A + c * (A @ A)) @ X
    if tall:
        X = X.transpose(-2, -1)
    return X.to(M.dtype)


class Muon(Optimizer):
    """Muon for 2-D parameters (see module docstring)."""

    def __init__(self, params: Any, lr: float = 0.03, momentum: float = 0.95, nesterov: bool = True,
                 weight_decay: float = 0.01, ns_iterations: int = 5, ns_coefficients: Optional[str] = None) -> None:
        super().__init__(params, dict(lr=lr, momentum=momentum, nesterov=nesterov, weight_decay=weight_decay,
                                      ns_iterations=ns_iterations))
        self._ns_coefficients = ns_coefficients
        resolve_ns_coefficients(ns_coefficients, ns_iterations)

    def state_dict(self) -> dict[str, Any]:
        sd = super().state_dict()
        sd["ns_coefficients"] = self._ns_coefficients
        return sd

    def load_state_dict(self, state_dict: dict[str, Any]) -> None:
        state_dict = dict(state_dict)
        coeff = state_dict.pop("ns_coefficients", None)
        super().load_state_dict(state_dict)
        if coeff is not None:
            if self._ns_coefficients is not None and self._ns_coefficients != coeff:
                logger.warning("Muon ns_coefficients: checkpoint has '%s', caller asked for '%s'; keeping the "
                               "checkpoint's.", coeff, self._ns_coefficients)
            self._ns_coefficients = coeff

    @torch.no_grad()
    def step(self, closure: Any = None) -> Any:
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, mom, wd = group["lr"], group["momentum"], group["weight_decay"]
            by_shape: dict[tuple[int, int], list[tuple[torch.Tensor, torch.Tensor]]] = {}
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["momentum_buffer"] = torch.zeros_like(p.grad)
                buf = st["momentum_buffer"]
                buf.mul_(mom).add_(p.grad)
                upd = mom * buf + p.grad if group["nesterov"] else buf.clone()
                if hasattr(p, "_tp_shard_dim"):
                    from ..parallel.tp import all_gather_along_dim
                    upd = all_gather_along_dim(upd, p._tp_shard_dim, p._tp_group)
                by_shape.setdefault(tuple(upd.shape), []).append((p, upd))
            for shape, items in by_shape.items():
                batch = torch.stack([u for _, u in items]) if len(items) > 1 else items[0][1]
                orth = newton_schulz_orthogonalize(batch, group["ns_iterations"], self._ns_coefficients)
                orth = orth.unbind(0) if len(items) > 1 else [orth]
                scale = max(1.0, (shape[0] / shape[1]) ** 0.5)
                for (p, _), o in zip(items, orth):
                    if hasattr(p, "_tp_shard_dim"):
                        n = p.shape[p._tp_shard_dim]
                        o = o.narrow(p._tp_shard_dim, p._tp_rank * n, n)
                    if wd > 0:
                        p.mul_(1 - lr * wd)
                    p.add_(o.to(p.dtype), alpha=-lr * scale)
        return loss


def split_params(model: torch.nn.Module) -> tuple[list, list]:
    """``(muon_params, adamw_params)`` by the reference rule, in ``named_parameters`` order."""
    muon, adamw = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        (muon if (p.ndim == 2 and "embed" not in name and "lm_head" not in name) else adamw).append(p)
    return muon, adamw


def build_hybrid_optimizer(model: torch.nn.Module, muon_lr: float = 0.03, muon_momentum: float = 0.95,
                           muon_weight_decay: float = 0.01, muon_ns_iterations: int = 5,
                           muon_ns_coefficients: Optional[str] = None, adamw_lr: float = 6e-4,
                           adamw_betas: tuple[float, float] = (0.9, 0.95),
                           adamw_weight_decay: float = 0.1) -> tuple[Muon, AdamW]:
    muon, adamw = split_params(model)
    nm, na = sum(p.numel() for p in muon), sum(p.numel() for p in adamw)
    import torch.distributed as dist
    if not (dist.is_available() and dist.is_initialized()) or dist.get_rank() == 0:
        print(f"Muon params:  {nm:>12,} ({nm / max(nm + na, 1) * 100:.1f}%)")
        print(f"AdamW params: {na:>12,} ({na / max(nm + na, 1) * 100:.1f}%)")
    return (Muon(muon, lr=muon_lr, momentum=muon_momentum, nesterov=True, weight_decay=muon_weight_decay,
                 ns_iterations=muon_ns_iterations, ns_coefficients=muon_ns_coefficients),
            AdamW(adamw, lr=adamw_lr, betas=adamw_betas, weight_decay=adamw_weight_decay))


class HybridScheduler:
    """Warmup-stable-decay multiplier applied to both optimizers' base learning rates.

    ``get_lr_multiplier(step)``: ``step/warmup`` during warmup, 1 until ``int(total*pct)``, then
    ``1-sqrt(p)``, ``1-p`` or a half cosine over the remaining steps.
    """

    def __init__(self, muon_opt: Any, adamw_opt: Any, warmup_steps: int = 2000, total_steps: int = 100000,
                 decay_start_pct: float = 0.90, decay_type: str = "sqrt") -> None:
        if decay_type not in ("sqrt", "linear", "cosine"):
            raise ValueError(f"Unknown decay type: {decay_type}")
        self.muon_opt, self.adamw_opt = muon_opt, adamw_opt
        self.warmup_steps, self.total_steps = warmup_steps, total_steps
        self.decay_start_step = int(total_steps * decay_start_pct)
        self.decay_type = decay_type
        self.muon_base_lr = muon_opt.defaults["lr"]
        self.adamw_base_lr = adamw_opt.defaults["lr"]

    def get_lr_multiplier(self, step: int) -> float:
        if step < self.warmup_steps:
            return step / self.warmup_steps
        if step < self.decay_start_step:
            return 1.0
        p = (step - self.decay_start_step) / max(self.total_steps - self.decay_start_step, 1)
        if self.decay_type == "sqrt":
            return 1.0 - p ** 0.5
        if self.decay_type == "linear":
            return 1.0 - p
        return 0.5 * (1 + math.cos(p * 3.14159))

    def step(self, step: int) -> None:
        m = self.get_lr_multiplier(step)
        for g in self.muon_opt.param_groups:
            g["lr"] = self.muon_base_lr * m
        for g in self.adamw_opt.param_groups:
            g["lr"] = self.adamw_base_lr * m

    def get_last_lr(self) -> dict[str, float]:
        return {"muon_lr": self.muon_opt.param_groups[0]["lr"] if self.muon_opt.param_groups else 0.0,
                "adamw_lr": self.adamw_opt.param_groups[0]["lr"] if self.adamw_opt.param_groups else 0.0}

    def state_dict(self) -> dict[str, Any]:
        return dict(warmup_steps=self.warmup_steps, total_steps=self.total_steps,
                    decay_start_step=self.decay_start_step, decay_type=self.decay_type,
                    muon_base_lr=self.muon_base_lr, adamw_base_lr=self.adamw_base_lr)


class NoOpOptimizer:
    """Stand-in for Muon under ``--adamw_only`` (``train.py:881-897``)."""

    param_groups: list[dict[str, Any]] = []
    defaults: dict[str, Any] = {"lr": 0.0}

    def step(self, closure: Any = None) -> None:
        return None

    def zero_grad(self, set_to_none: bool = False) -> None:
        return None

    def state_dict(self) -> dict[str, Any]:
        return {}

    def load_state_dict(self, state: dict[str, Any]) -> None:
        return None
