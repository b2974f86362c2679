"""Neural-cellular-automata pre-pre-training data.

Random "rule" networks drive multi-channel discrete grids; trajectories are serialised to the
same flat uint16 token format as language data.  Behaviour follows the reference generator
(``src/nca/generator.py``): rule = circular k x k perception conv -> ReLU -> n x (1x1 conv, ReLU)
-> 1x1 conv logits over ``d_state`` per channel, weights N(0, 0.5), biases N(0, 0.1)
(``:129-194``); a step adds ``identity_bias`` to the current state's logit, applies a
temperature softmax per cell and samples (``:254-275``); ``burn_in`` steps are discarded;
tokens are base-``d`` codes of 2x2 patches, ``START = d^4``, ``END = d^4 + 1``, one frame per
channel per time step (``:297-351``); rules are kept when the gzip ratio of a short rollout is
inside ``[0.4, 0.7]`` (``:354-459``).

The simulator and the tokeniser are batched tensor programs (no per-cell Python), so they run
unchanged on ``cuda`` for bulk generation.
"""
from __future__ import annotations

import argparse
import gzip
import logging
import random
import time
from dataclasses import dataclass
from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch
import torch.nn.functional as F

logger = logging.getLogger(__name__)


@dataclass
class NCAConfig:
    grid_size: int = 32
    d_state: int = 10
    n_groups: int = 4
    kernel_size: int = 3
    hidden_dim: int = 32
    num_hidden_layers: int = 2
    identity_bias: float = 1.0
    temperature: float = 0.5
    num_steps: int = 128
    burn_in: int = 10
    filter_enabled: bool = True
    gzip_lower: float = 0.4
    gzip_upper: float = 0.7
    filter_steps: int = 30
    patch_size: int = 2
    mixed_complexity: bool = True

    @property
    def vocab_size(self) -> int:
        return self.d_state ** (self.patch_size ** 2) + 2

    @property
    def patches_per_frame(self) -> int:
        return (self.grid_size // self.patch_size) ** 2

    @property
    def tokens_per_frame(self) -> int:
        return self.patches_per_frame + 2

    @property
    def tokens_per_timestep(self) -> int:
        return self.tokens_per_frame * self.n_groups

    @property
    def tokens_per_trajectory(self) -> int:
        return self.tokens_per_timestep * self.num_steps


class NCARule(torch.nn.Module):
    """One random automaton: ``(B, G*d, H, W)`` one-hot state -> next-state logits of the same shape."""

    def __init__(self, d_state: int, n_groups: int, kernel_size: int, hidden_dim: int, num_hidden_layers: int,
                 generator: Optional[torch.Generator] = None) -> None:
        super().__init__()
        self.d_state, self.n_groups, self.kernel_size = d_state, n_groups, kernel_size
        c = d_state * n_groups
        shapes = [(hidden_dim, c, kernel_size, kernel_size)] + [(hidden_dim, hidden_dim, 1, 1)] * num_hidden_layers \
            + [(c, hidden_dim, 1, 1)]
        self.weights = torch.nn.ParameterList()
        self.biases = torch.nn.ParameterList()
        for s in shapes:
            self.weights.append(torch.nn.Parameter(torch.randn(s, generator=generator) * 0.5, requires_grad=False))
            self.biases.append(torch.nn.Parameter(torch.randn(s[0], generator=generator) * 0.1, requires_grad=False))

    def forward(self, onehot: torch.Tensor) -> torch.Tensor:
        pad = self.kernel_size // 2
        x = F.pad(onehot, (pad, pad, pad, pad), mode="circular") if pad else onehot
        n = len(self.weights)
        for i, (w, b) in enumerate(zip(self.weights, self.biases)):
            x = F.conv2d(x, w, b)
            if i < n - 1:
                x = F.relu(x)
        return x


def sample_rule_config(config: NCAConfig, rng: Optional[random.Random] = None) -> dict[str, Any]:
    """Rule architecture and dynamics drawn from the design space (fixed values without mixing)."""
    if not config.mixed_complexity:
        return dict(kernel_size=config.kernel_size, hidden_dim=config.hidden_dim,
                    num_hidden_layers=config.num_hidden_layers, identity_bias=config.identity_bias,
                    temperature=config.temperature)
    r = rng or random
    return dict(kernel_size=r.choice([3, 5]), hidden_dim=r.choice([16, 32, 48]), num_hidden_layers=r.choice([1, 2, 3]),
                identity_bias=r.uniform(0.5, 2.0), temperature=r.uniform(0.3, 1.0))


@torch.no_grad()
def nca_step(rule: NCARule, state: torch.Tensor, d: int, identity_bias: float, temperature: float,
             generator: Optional[torch.Generator] = None) -> torch.Tensor:
    """``state (B,G,H,W)`` integer -> next state, sampled per cell."""
    B, G, H, W = state.shape
    onehot = F.one_hot(state.long(), d).permute(0, 1, 4, 2, 3).reshape(B, G * d, H, W).float()
    logits = rule(onehot)
    if identity_bias > 0:
        logits = logits + identity_bias * onehot
    flat = logits.reshape(B, G, d, H, W).permute(0, 1, 3, 4, 2).reshape(-1, d)
    probs = torch.softmax(flat / max(temperature, 1e-6), dim=-1)
    return torch.multinomial(probs, 1, generator=generator).reshape(B, G, H, W)


@torch.no_grad()
def simulate_trajectory(rule: NCARule, grid_size: int, d_state: int, n_groups: int, num_steps: int, burn_in: int,
                        identity_bias: float, temperature: float, batch_size: int = 1,
                        device: torch.device | str = "cpu", generator: Optional[torch.Generator] = None
                        ) -> torch.Tensor:
    """Returns ``(batch, num_steps, n_groups, H, W)`` integer states."""
    device = torch.device(device)
    state = torch.randint(0, d_state, (batch_size, n_groups, grid_size, grid_size), device=device, generator=generator)
    for _ in range(burn_in):
        state = nca_step(rule, state, d_state, identity_bias, temperature, generator)
    traj = torch.empty(batch_size, num_steps, n_groups, grid_size, grid_size, dtype=torch.long, device=device)
    for t in range(num_steps):
        traj[:, t] = state
        state = nca_step(rule, state, d_state, identity_bias, temperature, generator)
    return traj


def tokenize_trajectory(trajectory: torch.Tensor, d_state: int, patch_size: int) -> np.ndarray:
    """``(B,T,G,H,W)`` states -> flat uint16 tokens: per time step and channel
    ``[START, patch codes row-major, END]``; a patch code is ``sum_i cell_i * d^i`` over the
    row-major cells of the patch."""
    B, T, G, H, W = trajectory.shape
    ps, d = patch_size, d_state
    nh, nw = H // ps, W // ps
    x = trajectory[..., : nh * ps, : nw * ps].reshape(B, T, G, nh, ps, nw, ps).permute(0, 1, 2, 3, 5, 4, 6)
    x = x.reshape(B, T, G, nh * nw, ps * ps).long()
    powers = torch.tensor([d ** i for i in range(ps * ps)], device=x.device, dtype=torch.long)
    codes = (x * powers).sum(-1)
    start = torch.full((B, T, G, 1), d ** (ps * ps), dtype=torch.long, device=x.device)
    frames = torch.cat([start, codes, start + 1], dim=-1)
    return frames.reshape(-1).cpu().numpy().astype(np.uint16)


def compute_gzip_complexity(tokens: np.ndarray) -> float:
    raw = tokens.tobytes()
    return len(gzip.compress(raw)) / max(len(raw), 1)


def evaluate_rule_complexity(rule: NCARule, config: NCAConfig, params: dict[str, Any], device: Any,
                             eval_sims: int = 4) -> float:
    traj = simulate_trajectory(rule, config.grid_size, config.d_state, config.n_groups, config.filter_steps,
                               config.burn_in, params["identity_bias"], params["temperature"], eval_sims, device)
    return compute_gzip_complexity(tokenize_trajectory(traj, config.d_state, config.patch_size))


def generate_and_filter_rules(config: NCAConfig, num_rules: int, device: Any, eval_sims: int = 4,
                              max_candidates: Optional[int] = None) -> list[tuple[NCARule, dict[str, Any]]]:
    """Draw rules until ``num_rules`` pass the complexity band (Class-IV, edge of chaos)."""
    accepted: list[tuple[NCARule, dict[str, Any]]] = []
    tested = 0
    t0 = time.time()
    while len(accepted) < num_rules and (max_candidates is None or tested < max_candidates):
        params = sample_rule_config(config)
        rule = NCARule(config.d_state, config.n_groups, params["kernel_size"], params["hidden_dim"],
                       params["num_hidden_layers"]).to(device)
        tested += 1
        if config.filter_enabled:
            ratio = evaluate_rule_complexity(rule, config, params, device, eval_sims)
            if not (config.gzip_lower <= ratio <= config.gzip_upper):
                continue
        accepted.append((rule, params))
    logger.info("Rule generation: %d accepted from %d candidates (%.0f%%, %.1fs)", len(accepted), tested,
                100 * len(accepted) / max(tested, 1), time.time() - t0)
    return accepted


def generate_nca_dataset(config: NCAConfig, output_path: str | Path, max_tokens: int = 300_000_000,
                         num_rules: int = 5000, sims_per_rule: int = 8, device: Any = "cpu") -> int:
    """Rules -> trajectories -> tokens -> flat uint16 file (readable by ``TokenizedDataset``).
    Returns the number of tokens written (truncated to ``max_tokens``)."""
    output_path = Path(output_path)
    output_path.parent.mkdir(parents=True, exist_ok=True)
    logger.info("NCA dataset: grid %dx%d, %d states, %d channels, %d tok/timestep, %d tok/trajectory",
                config.grid_size, config.grid_size, config.d_state, config.n_groups, config.tokens_per_timestep,
                config.tokens_per_trajectory)
    rules = generate_and_filter_rules(config, num_rules, device)
    total = 0
    t0 = time.time()
    with open(output_path, "wb") as fh:
        for rule, params in rules:
            traj = simulate_trajectory(rule, config.grid_size, config.d_state, config.n_groups, config.num_steps,
                                       config.burn_in, params["identity_bias"], params["temperature"], sims_per_rule,
                                       device)
            toks = tokenize_trajectory(traj, config.d_state, config.patch_size)
            fh.write(toks.tobytes())
            total += len(toks)
            if total >= max_tokens:
                break
    if total > max_tokens:
        with open(output_path, "r+b") as fh:
            fh.truncate(max_tokens * 2)
        total = max_tokens
    logger.info("Done: %d rules, %.1fM tokens, %.1fs", len(rules), total / 1e6, time.time() - t0)
    return total


def verify_file(path: str | Path, config: Optional[NCAConfig] = None) -> dict[str, Any]:
    """Size and id range of a written token file (and, with a configuration, whether every id is in its vocabulary)."""
    arr = np.memmap(path, dtype=np.uint16, mode="r")
    out: dict[str, Any] = {"tokens": int(len(arr)), "max_id": int(arr.max()) if len(arr) else 0,
                           "min_id": int(arr.min()) if len(arr) else 0}
    if config is not None:
        out["in_vocab"] = bool(out["max_id"] < config.vocab_size)
        out["whole_timesteps"] = int(len(arr) // config.tokens_per_timestep)
    return out


def main(argv: Optional[list[str]] = None) -> None:
    """Command line with the reference's flags (``src/nca/generator.py:576-658``); ``--max_tokens`` is kept as a second
    name of ``--tokens``, and ``--verify`` takes an optional path (without one it checks the file just written)."""
    ap = argparse.ArgumentParser(description="Generate NCA pre-pre-training tokens")
    ap.add_argument("--output", default=None)
    ap.add_argument("--tokens", "--max_tokens", dest="tokens", type=int, default=300_000_000)
    ap.add_argument("--num_rules", type=int, default=5000)
    ap.add_argument("--sims_per_rule", type=int, default=8)
    ap.add_argument("--grid_size", type=int, default=32)
    ap.add_argument("--d_state", type=int, default=10)
    ap.add_argument("--n_groups", type=int, default=4)
    ap.add_argument("--kernel_size", type=int, default=3, choices=[3, 5])
    ap.add_argument("--hidden_dim", type=int, default=32)
    ap.add_argument("--num_hidden_layers", type=int, default=2)
    ap.add_argument("--identity_bias", type=float, default=1.0)
    ap.add_argument("--temperature", type=float, default=0.5)
    ap.add_argument("--gzip_lower", type=float, default=0.4)
    ap.add_argument("--gzip_upper", type=float, default=0.7)
    ap.add_argument("--no_filter", action="store_true")
    ap.add_argument("--no_mixed", action="store_true")
    ap.add_argument("--num_steps", type=int, default=128)
    ap.add_argument("--burn_in", type=int, default=10)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--verify", nargs="?", const="", default=None,
                    help="check a token file: the given path, or the file just written when no path follows")
    a = ap.parse_args(argv)
    logging.basicConfig(level=logging.INFO, format="%(asctime)s %(message)s")
    cfg = NCAConfig(grid_size=a.grid_size, d_state=a.d_state, n_groups=a.n_groups, kernel_size=a.kernel_size,
                    hidden_dim=a.hidden_dim, num_hidden_layers=a.num_hidden_layers, identity_bias=a.identity_bias,
                    temperature=a.temperature, num_steps=a.num_steps, burn_in=a.burn_in, filter_enabled=not a.no_filter,
                    gzip_lower=a.gzip_lower, gzip_upper=a.gzip_upper, mixed_complexity=not a.no_mixed)
    if a.verify:                                    # a path: only check that file
        logger.info("verify %s: %s", a.verify, verify_file(a.verify, cfg))
        return
    if not a.output:
        ap.error("--output is required unless --verify names a file")
    random.seed(a.seed)
    torch.manual_seed(a.seed)
    n = generate_nca_dataset(cfg, a.output, a.tokens, a.num_rules, a.sims_per_rule, a.device)
    if a.verify is not None:
        rep = verify_file(a.output, cfg)
        logger.info("verify: %s -> %s", rep, "OK" if rep["tokens"] == n and rep["in_vocab"] else "MISMATCH")


if __name__ == "__main__":
    main()
