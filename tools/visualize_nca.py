#!/usr/bin/env python
"""Render a few NCA trajectories as text frames (or PNG strips when matplotlib is installed) to
eyeball the dynamics of sampled rules:  python tools/visualize_nca.py --rules 3 --steps 6"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.nca.generator import (NCAConfig, NCARule, compute_gzip_complexity, sample_rule_config,  # noqa: E402
                                         simulate_trajectory, tokenize_trajectory)


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--rules", type=int, default=3)
    ap.add_argument("--steps", type=int, default=6)
    ap.add_argument("--grid", type=int, default=16)
    ap.add_argument("--png", default="")
    a = ap.parse_args()
    cfg = NCAConfig(grid_size=a.grid, num_steps=a.steps)
    glyph = " .:-=+*#%@"
    for r in range(a.rules):
        p = sample_rule_config(cfg)
        rule = NCARule(cfg.d_state, cfg.n_groups, p["kernel_size"], p["hidden_dim"], p["num_hidden_layers"])
        traj = simulate_trajectory(rule, cfg.grid_size, cfg.d_state, cfg.n_groups, a.steps, cfg.burn_in,
                                   p["identity_bias"], p["temperature"])
        ratio = compute_gzip_complexity(tokenize_trajectory(traj, cfg.d_state, cfg.patch_size))
        print(f"rule {r}: {p} gzip={ratio:.3f}")
        if a.png:
            try:
                import matplotlib
                matplotlib.use("Agg")
                import matplotlib.pyplot as plt
                fig, axes = plt.subplots(1, a.steps, figsize=(2 * a.steps, 2))
                for t, ax in enumerate(axes):
                    ax.imshow(traj[0, t, 0].numpy(), cmap="viridis"); ax.axis("off")
                fig.savefig(f"{a.png}_rule{r}.png", dpi=100); plt.close(fig)
                continue
            except ImportError:
                print("matplotlib not installed: text frames instead")
        for t in range(a.steps):
            print(f" t={t}")
            for row in traj[0, t, 0].tolist():
                print("  " + "".join(glyph[v % len(glyph)] for v in row))


if __name__ == "__main__":
    main()
