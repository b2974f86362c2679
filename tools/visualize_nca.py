#!/usr/bin/env python
"""Pictures of NCA dynamics, to judge a rule set or a generated token file by eye.

    python tools/visualize_nca.py --n-rules 6 --output-dir outputs/nca_viz          # sample rules, simulate, draw
    python tools/visualize_nca.py --from-data data/nca.bin --output-dir outputs/nca_viz   # decode a token file

For every sampled rule: a grid image (time steps left to right, one row per channel group), a
strip of evenly spaced frames of channel 0, a space-time image (one spatial row of every group
followed through ALL time steps: time runs left to right, space top to bottom - gliders show as
diagonals, frozen rules as horizontal stripes, noise as static), the rule's hyper-parameters and
its gzip complexity (the Class-IV filter keeps ratios in [0.4, 0.7]); a summary text file lists
them all.  ``--complexity-batch N`` also samples N more rules (short runs), and writes the
distribution of their gzip ratios as a histogram image and as numbers: how many rules the filter
would keep.  With ``--from-data`` the uint16 tokens are decoded back into grids (patch codes ->
cells, frames delimited by START/END) and the first trajectories are drawn the same way.

Images are written as PNG by a small encoder in this file (zlib only), so the tool has no
plotting dependency; states are coloured with an evenly spaced hue wheel, one colour per state
(the reference's tool does the same with matplotlib: ``scripts/utils/visualize_nca.py``).
"""
from __future__ import annotations

import argparse
import colorsys
import os
import struct
import sys
import zlib

import numpy as np
import torch

sys.path.insert(0, os.path.join(os.path.dirname(os.path.abspath(__file__)), ".."))
from kotodama_b200.nca.generator import (NCAConfig, NCARule, compute_gzip_complexity, sample_rule_config,  # noqa: E402
                                         simulate_trajectory, tokenize_trajectory)


def palette(n_states: int) -> np.ndarray:
    """One RGB colour per state: state 0 dark, the rest around the hue wheel."""
    cols = [(16, 16, 24)]
    for i in range(1, n_states):
        r, g, b = colorsys.hsv_to_rgb((i - 1) / max(n_states - 1, 1), 0.75, 0.95)
        cols.append((int(255 * r), int(255 * g), int(255 * b)))
    return np.asarray(cols, dtype=np.uint8)


def write_png(path: str, rgb: np.ndarray) -> None:
    """Minimal PNG writer: ``rgb[H, W, 3]`` uint8, no interlace, one IDAT chunk."""
    h, w, _ = rgb.shape
    raw = b"".join(b"\x00" + rgb[y].tobytes() for y in range(h))

    def chunk(tag: bytes, data: bytes) -> bytes:
        return struct.pack(">I", len(data)) + tag + data + struct.pack(">I", zlib.crc32(tag + data) & 0xFFFFFFFF)
    with open(path, "wb") as fh:
        fh.write(b"\x89PNG\r\n\x1a\n" + chunk(b"IHDR", struct.pack(">IIBBBBB", w, h, 8, 2, 0, 0, 0))
                 + chunk(b"IDAT", zlib.compress(raw, 6)) + chunk(b"IEND", b""))


def tile(frames: np.ndarray, pal: np.ndarray, cell: int, gap: int = 2) -> np.ndarray:
    """``frames[R, C, H, W]`` of states -> one image: R rows and C columns of grids, ``cell`` pixels per cell."""
    R, C, H, W = frames.shape
    out = np.full((R * (H * cell + gap) + gap, C * (W * cell + gap) + gap, 3), 40, dtype=np.uint8)
    for r in range(R):
        for c in range(C):
            img = pal[frames[r, c] % len(pal)].repeat(cell, 0).repeat(cell, 1)
            y, x = gap + r * (H * cell + gap), gap + c * (W * cell + gap)
            out[y:y + H * cell, x:x + W * cell] = img
    return out


def space_time(traj: np.ndarray, pal: np.ndarray, cell: int = 4, gap: int = 2) -> np.ndarray:
    """``traj[T, G, H, W]`` -> one image with a band per group: the middle row of the grid at every time step
    (x = time, y = position in the row)."""
    T, G, H, W = traj.shape
    out = np.full((G * (W * cell + gap) + gap, T * cell + 2 * gap, 3), 40, dtype=np.uint8)
    for g in range(G):
        band = pal[traj[:, g, H // 2, :].T % len(pal)].repeat(cell, 0).repeat(cell, 1)      # [W, T] -> pixels
        y = gap + g * (W * cell + gap)
        out[y:y + W * cell, gap:gap + T * cell] = band
    return out


def histogram(values: list[float], lo: float, hi: float, keep: tuple[float, float], bins: int = 30, w: int = 14, h: int = 160) -> np.ndarray:
    """Bar chart of ``values`` over [lo, hi]; bars inside ``keep`` are drawn in the kept colour."""
    counts, edges = np.histogram(np.clip(values, lo, hi), bins=bins, range=(lo, hi))
    top = max(int(counts.max()), 1)
    img = np.full((h + 12, bins * w + 8, 3), 24, dtype=np.uint8)
    for i, c in enumerate(counts):
        mid = (edges[i] + edges[i + 1]) / 2
        colour = (90, 200, 120) if keep[0] <= mid <= keep[1] else (200, 110, 90)
        bar = int(round(c / top * h))
        if bar:
            img[6 + h - bar:6 + h, 4 + i * w + 1:4 + (i + 1) * w - 1] = colour
    for edge in keep:                                     # thin lines at the filter's limits
        x = 4 + int((edge - lo) / (hi - lo) * bins * w)
        img[4:8 + h, x:x + 1] = (230, 230, 230)
    return img


def draw_trajectory(traj: np.ndarray, d_state: int, prefix: str, n_frames: int = 8) -> None:
    """``traj[T, G, H, W]``: grid image (groups x sampled time steps), a strip of channel 0, a space-time image."""
    T, G, H, W = traj.shape
    pal = palette(d_state)
    steps = np.unique(np.linspace(0, T - 1, min(n_frames, T)).astype(int))
    cell = max(2, 128 // H)
    write_png(prefix + "_grid.png", tile(traj[steps].transpose(1, 0, 2, 3), pal, cell))
    write_png(prefix + "_strip.png", tile(traj[steps, 0][None], pal, cell * 2))
    write_png(prefix + "_spacetime.png", space_time(traj, pal, max(2, 96 // W)))


def from_generator(a: argparse.Namespace) -> None:
    cfg = NCAConfig(grid_size=a.grid, num_steps=a.steps)
    gen = torch.Generator(device="cpu").manual_seed(a.seed)
    import random
    rng = random.Random(a.seed)
    lines = []
    for r in range(a.n_rules):
        p = sample_rule_config(cfg, rng)
        torch.manual_seed(a.seed + r)
        rule = NCARule(cfg.d_state, cfg.n_groups, p["kernel_size"], p["hidden_dim"], p["num_hidden_layers"]).to(a.device)
        traj = simulate_trajectory(rule, cfg.grid_size, cfg.d_state, cfg.n_groups, cfg.num_steps, cfg.burn_in,
                                   p["identity_bias"], p["temperature"], device=a.device,
                                   generator=gen if a.device == "cpu" else None)
        toks = tokenize_trajectory(traj, cfg.d_state, cfg.patch_size)
        ratio = compute_gzip_complexity(toks)
        verdict = "kept" if cfg.gzip_lower <= ratio <= cfg.gzip_upper else "filtered out"
        states = traj[0].cpu().numpy()
        change = float((states[1:] != states[:-1]).mean()) if len(states) > 1 else 0.0
        draw_trajectory(states, cfg.d_state, os.path.join(a.output_dir, f"rule{r:02d}"), a.frames)
        line = (f"rule {r:02d}: kernel {p['kernel_size']} hidden {p['hidden_dim']}x{p['num_hidden_layers']} "
                f"identity_bias {p['identity_bias']:.2f} temperature {p['temperature']:.2f} | gzip {ratio:.3f} ({verdict}) "
                f"| cells changing per step {change:.3f} | {len(toks)} tokens")
        print(line)
        lines.append(line)
    if a.complexity_batch > 0:
        short = NCAConfig(grid_size=a.grid, num_steps=min(a.steps, 32))
        ratios = []
        for r in range(a.complexity_batch):
            p = sample_rule_config(short, rng)
            torch.manual_seed(a.seed + 1000 + r)
            rule = NCARule(short.d_state, short.n_groups, p["kernel_size"], p["hidden_dim"], p["num_hidden_layers"]).to(a.device)
            traj = simulate_trajectory(rule, short.grid_size, short.d_state, short.n_groups, short.num_steps, short.burn_in,
                                       p["identity_bias"], p["temperature"], device=a.device,
                                       generator=gen if a.device == "cpu" else None)
            ratios.append(compute_gzip_complexity(tokenize_trajectory(traj, short.d_state, short.patch_size)))
        kept = sum(cfg.gzip_lower <= x <= cfg.gzip_upper for x in ratios)
        write_png(os.path.join(a.output_dir, "complexity_histogram.png"),
                  histogram(ratios, 0.0, 1.0, (cfg.gzip_lower, cfg.gzip_upper)))
        line = (f"complexity of {len(ratios)} sampled rules: min {min(ratios):.3f} median {float(np.median(ratios)):.3f} "
                f"max {max(ratios):.3f}; the filter [{cfg.gzip_lower}, {cfg.gzip_upper}] keeps {kept} ({100 * kept / len(ratios):.0f} %)")
        print(line)
        lines.append(line)
    with open(os.path.join(a.output_dir, "summary.txt"), "w") as fh:
        fh.write("\n".join(lines) + "\n")


def decode_tokens(tokens: np.ndarray, cfg: NCAConfig) -> np.ndarray:
    """Flat tokens -> ``[n_frames, H, W]`` grids (every START..END frame is one channel of one time step)."""
    d, ps = cfg.d_state, cfg.patch_size
    start = d ** (ps * ps)
    per = cfg.tokens_per_frame
    n = len(tokens) // per
    fr = tokens[: n * per].reshape(n, per).astype(np.int64)
    good = (fr[:, 0] == start) & (fr[:, -1] == start + 1)
    codes = fr[good][:, 1:-1]
    side = cfg.grid_size // ps
    cells = np.stack([(codes // d ** i) % d for i in range(ps * ps)], -1)           # [n, patches, ps*ps]
    grids = cells.reshape(-1, side, side, ps, ps).transpose(0, 1, 3, 2, 4).reshape(-1, side * ps, side * ps)
    return grids


def from_data(a: argparse.Namespace) -> None:
    cfg = NCAConfig(grid_size=a.grid, num_steps=a.steps)
    toks = np.fromfile(a.from_data, dtype="<u2", count=a.trajectories * cfg.tokens_per_trajectory)
    grids = decode_tokens(toks, cfg)
    per_traj = cfg.num_steps * cfg.n_groups
    n = len(grids) // per_traj
    print(f"{a.from_data}: {len(toks)} tokens read, {len(grids)} well-formed frames, {n} whole trajectories")
    for k in range(n):
        traj = grids[k * per_traj:(k + 1) * per_traj].reshape(cfg.num_steps, cfg.n_groups, cfg.grid_size, cfg.grid_size)
        draw_trajectory(traj, cfg.d_state, os.path.join(a.output_dir, f"data{k:02d}"), a.frames)
        ratio = compute_gzip_complexity(toks[k * cfg.tokens_per_trajectory:(k + 1) * cfg.tokens_per_trajectory])
        print(f"trajectory {k:02d}: gzip {ratio:.3f}")


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__.split("\n\n")[0])
    ap.add_argument("--output-dir", default="outputs/nca_viz")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--n-rules", type=int, default=6)
    ap.add_argument("--from-data", default=None, help="decode and draw a generated .bin instead of sampling rules")
    ap.add_argument("--trajectories", type=int, default=4, help="with --from-data: how many trajectories to draw")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--grid", type=int, default=32)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--frames", type=int, default=8, help="time steps shown per image")
    ap.add_argument("--complexity-batch", type=int, default=0, help="also sample this many rules and draw the distribution of their gzip ratios")
    a = ap.parse_args()
    os.makedirs(a.output_dir, exist_ok=True)
    if a.from_data:
        from_data(a)
    else:
        from_generator(a)
    print("images in", a.output_dir)


if __name__ == "__main__":
    main()
