"""Plot defaults and a small dependency-free plotting layer for the analysis tracks.

Two parts:

* **Style**: one colour, marker and short label per run name, stable across all figures of a report (a run
  keeps its colour whatever subset of runs a figure shows), labels for the weight types, and `apply_style`
  for matplotlib where it is installed.  Same role as the reference's ``src/eval/plot_utils.py``; names
  that are not in the table get a colour from a hash of the name, so ad-hoc run names stay stable too.
* **SVG figures without matplotlib**: `line_chart`, `scatter`, `heatmap`, `bar_chart` return a complete
  ``<svg>`` document as a string (axes with ticks, legend, labels).  The visualisers fall back to them when
  matplotlib cannot be imported, so every track produces pictures on a bare Python install; the report embeds
  the files inline.
"""
from __future__ import annotations

import html
import math
import zlib
from typing import Any, Iterable, Optional, Sequence

PALETTE = ["#1f77b4", "#ff7f0e", "#2ca02c", "#d62728", "#9467bd", "#8c564b", "#e377c2", "#7f7f7f", "#bcbd22", "#17becf"]
MARKERS = ["o", "s", "^", "D", "v", "P", "*", "X", "H", "<"]

# runs that appear in most comparisons keep a fixed place in the palette
RUN_STYLE: dict[str, tuple[str, str, str]] = {       # name -> (colour, marker, short label)
    "proxy-adamw": ("#7f7f7f", "s", "AdamW"),
    "proxy-muon": ("#1f77b4", "o", "Muon"),
    "proxy-muon-003": ("#aec7e8", "^", "Muon-3"),
    "proxy-nca": ("#2ca02c", "D", "NCA"),
    "proxy-attnres": ("#ff7f0e", "P", "AttnRes"),
    "proxy-nca-attnres": ("#d62728", "*", "NCA+AR"),
    "lang-baseline": ("#9467bd", "X", "Baseline"),
    "lang-ddv1": ("#e377c2", "H", "DD-v1"),
}
WEIGHT_TYPE_LABELS = {"q_proj": "Q", "k_proj": "K", "v_proj": "V", "o_proj": "O", "gate_proj": "gate", "up_proj": "up", "down_proj": "down"}
WEIGHT_TYPE_COLORS = {"q_proj": "#1f77b4", "k_proj": "#ff7f0e", "v_proj": "#2ca02c", "o_proj": "#d62728", "gate_proj": "#9467bd",
                      "up_proj": "#8c564b", "down_proj": "#e377c2"}


def run_color(name: str) -> str:
    if name.lower() in RUN_STYLE:
        return RUN_STYLE[name.lower()][0]
    return PALETTE[zlib.crc32(name.encode()) % len(PALETTE)]


def run_marker(name: str) -> str:
    if name.lower() in RUN_STYLE:
        return RUN_STYLE[name.lower()][1]
    return MARKERS[zlib.crc32(name.encode()) % len(MARKERS)]


def run_label(name: str, max_len: int = 14) -> str:
    if name.lower() in RUN_STYLE:
        return RUN_STYLE[name.lower()][2]
    return name if len(name) <= max_len else name[: max_len - 1] + "…"


def apply_style(plt: Any, dark: bool = False) -> None:
    """Common matplotlib settings of the analysis figures."""
    plt.rcParams.update({"figure.dpi": 120, "axes.grid": True, "grid.alpha": 0.25, "axes.spines.top": False,
                         "axes.spines.right": False, "font.size": 9, "legend.fontsize": 7, "lines.linewidth": 1.4,
                         "lines.markersize": 3})
    if dark:
        plt.style.use("dark_background")


# ------------------------------------------------------------------------------ SVG figures
def _finite(vals: Iterable[float]) -> list[float]:
    return [float(v) for v in vals if v is not None and math.isfinite(float(v))]


def _ticks(lo: float, hi: float, n: int = 5) -> list[float]:
    """Round tick positions covering [lo, hi]."""
    if hi <= lo:
        return [lo]
    raw = (hi - lo) / n
    mag = 10 ** math.floor(math.log10(raw))
    step = min((m * mag for m in (1, 2, 2.5, 5, 10)), key=lambda s: abs(s - raw))
    first = math.ceil(lo / step) * step
    out, v = [], first
    while v <= hi + 1e-9 * (hi - lo):
        out.append(round(v, 10))
        v += step
    return out or [lo]


def _fmt(v: float) -> str:
    return f"{v:.3g}" if abs(v) < 1e4 else f"{v:.2e}"


class _Frame:
    """Plot area with data -> pixel mapping, axes and labels."""

    def __init__(self, xs: Sequence[float], ys: Sequence[float], w: int, h: int, title: str, xlabel: str, ylabel: str,
                 legend_w: int = 0, x_ticks: bool = True, pad_x: bool = False) -> None:
        self.w, self.h = w, h
        self.l, self.r, self.t, self.b = 52, 12 + legend_w, 26 if title else 10, 34
        fx, fy = _finite(xs) or [0.0, 1.0], _finite(ys) or [0.0, 1.0]
        self.x0, self.x1, self.y0, self.y1 = min(fx), max(fx), min(fy), max(fy)
        if self.x1 == self.x0:
            self.x0, self.x1 = self.x0 - 0.5, self.x1 + 0.5
        if self.y1 == self.y0:
            self.y0, self.y1 = self.y0 - 0.5, self.y1 + 0.5
        pad = 0.04 * (self.y1 - self.y0)
        self.y0, self.y1 = self.y0 - pad, self.y1 + pad
        if pad_x:
            pad = 0.06 * (self.x1 - self.x0)
            self.x0, self.x1 = self.x0 - pad, self.x1 + pad
        self.parts = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}" '
                      f'font-family="sans-serif" font-size="10"><rect width="{w}" height="{h}" fill="white"/>']
        if title:
            self.parts.append(f'<text x="{w / 2:.0f}" y="15" text-anchor="middle" font-size="12">{html.escape(title)}</text>')
        for tx in (_ticks(self.x0, self.x1) if x_ticks else []):
            px = self.px(tx)
            self.parts.append(f'<line x1="{px:.1f}" y1="{self.t}" x2="{px:.1f}" y2="{h - self.b}" stroke="#e6e6e6"/>'
                              f'<text x="{px:.1f}" y="{h - self.b + 12}" text-anchor="middle">{_fmt(tx)}</text>')
        for ty in _ticks(self.y0, self.y1):
            py = self.py(ty)
            self.parts.append(f'<line x1="{self.l}" y1="{py:.1f}" x2="{w - self.r}" y2="{py:.1f}" stroke="#e6e6e6"/>'
                              f'<text x="{self.l - 4}" y="{py + 3:.1f}" text-anchor="end">{_fmt(ty)}</text>')
        self.parts.append(f'<rect x="{self.l}" y="{self.t}" width="{w - self.l - self.r}" height="{h - self.t - self.b}" '
                          'fill="none" stroke="#888"/>')
        if xlabel:
            self.parts.append(f'<text x="{(self.l + w - self.r) / 2:.0f}" y="{h - 6}" text-anchor="middle">{html.escape(xlabel)}</text>')
        if ylabel:
            self.parts.append(f'<text x="12" y="{(self.t + h - self.b) / 2:.0f}" text-anchor="middle" '
                              f'transform="rotate(-90 12 {(self.t + h - self.b) / 2:.0f})">{html.escape(ylabel)}</text>')

    def px(self, x: float) -> float:
        return self.l + (x - self.x0) / (self.x1 - self.x0) * (self.w - self.l - self.r)

    def py(self, y: float) -> float:
        return self.h - self.b - (y - self.y0) / (self.y1 - self.y0) * (self.h - self.t - self.b)

    def legend(self, entries: list[tuple[str, str]]) -> None:
        x = self.w - self.r + 8
        for i, (label, colour) in enumerate(entries):
            y = self.t + 10 + 14 * i
            self.parts.append(f'<line x1="{x}" y1="{y - 3}" x2="{x + 14}" y2="{y - 3}" stroke="{colour}" stroke-width="2"/>'
                              f'<text x="{x + 18}" y="{y}">{html.escape(label)}</text>')

    def done(self) -> str:
        return "".join(self.parts) + "</svg>"


def line_chart(series: dict[str, Sequence[float]], title: str = "", xlabel: str = "", ylabel: str = "",
               x: Optional[Sequence[float]] = None, colors: Optional[dict[str, str]] = None, dashed: Iterable[str] = (),
               w: int = 520, h: int = 300) -> str:
    """One polyline per entry of ``series`` (gaps at None / NaN), with point markers and a legend."""
    names = list(series)
    xs_all = list(x) if x is not None else list(range(max((len(v) for v in series.values()), default=1)))
    ys_all = [v for s in series.values() for v in s]
    legend_w = 0 if len(names) <= 1 else 24 + 6 * max(len(run_label(n, 18)) for n in names)
    f = _Frame(xs_all, ys_all, w, h, title, xlabel, ylabel, legend_w)
    dashed = set(dashed)
    entries = []
    for name in names:
        colour = (colors or {}).get(name) or run_color(name)
        entries.append((run_label(name, 18), colour))
        seg: list[str] = []
        pts: list[str] = []

        def flush() -> None:
            if len(seg) > 1:
                dash = ' stroke-dasharray="4 3"' if name in dashed else ""
                f.parts.append(f'<polyline fill="none" stroke="{colour}" stroke-width="1.5"{dash} points="{" ".join(seg)}"/>')
            seg.clear()
        for i, v in enumerate(series[name]):
            if v is None or not math.isfinite(float(v)) or i >= len(xs_all):
                flush()
                continue
            px, py = f.px(float(xs_all[i])), f.py(float(v))
            seg.append(f"{px:.1f},{py:.1f}")
            pts.append(f'<circle cx="{px:.1f}" cy="{py:.1f}" r="2" fill="{colour}"/>')
        flush()
        if len(pts) <= 80:
            f.parts.extend(pts)
    if len(names) > 1:
        f.legend(entries)
    return f.done()


def scatter(points: Sequence[Sequence[float]], labels: Optional[Sequence[str]] = None, title: str = "", xlabel: str = "",
            ylabel: str = "", connect: str = "", arrows: Optional[Sequence[tuple[int, int]]] = None,
            ghosts: Optional[Sequence[Sequence[float]]] = None, colors: Optional[Sequence[str]] = None, w: int = 440, h: int = 420) -> str:
    """2-D points with optional text labels.  ``connect``: "path" joins them in order, "loop" also closes the
    path; ``arrows``: index pairs drawn as arrows; ``ghosts``: a second point set drawn faintly, each joined to the
    point of the same index (e.g. true map positions)."""
    pts = [(float(p[0]), float(p[1])) for p in points]
    allp = pts + [(float(g[0]), float(g[1])) for g in (ghosts or [])]
    f = _Frame([p[0] for p in allp], [p[1] for p in allp], w, h, title, xlabel, ylabel, pad_x=True)
    n = len(pts)
    if ghosts:
        for (x0, y0), g in zip(pts, ghosts):
            f.parts.append(f'<line x1="{f.px(x0):.1f}" y1="{f.py(y0):.1f}" x2="{f.px(float(g[0])):.1f}" y2="{f.py(float(g[1])):.1f}" '
                           'stroke="#cccccc" stroke-width="0.7"/>'
                           f'<circle cx="{f.px(float(g[0])):.1f}" cy="{f.py(float(g[1])):.1f}" r="2.5" fill="#cccccc"/>')
    if connect in ("path", "loop") and n > 1:
        order = list(range(n)) + ([0] if connect == "loop" else [])
        f.parts.append('<polyline fill="none" stroke="#999" stroke-width="0.8" points="'
                       + " ".join(f"{f.px(pts[i][0]):.1f},{f.py(pts[i][1]):.1f}" for i in order) + '"/>')
    if arrows:
        f.parts.append('<defs><marker id="ah" markerWidth="6" markerHeight="6" refX="5" refY="3" orient="auto">'
                       '<path d="M0,0 L6,3 L0,6 z" fill="#777"/></marker></defs>')
        for a, b in arrows:
            f.parts.append(f'<line x1="{f.px(pts[a][0]):.1f}" y1="{f.py(pts[a][1]):.1f}" x2="{f.px(pts[b][0]):.1f}" '
                           f'y2="{f.py(pts[b][1]):.1f}" stroke="#777" stroke-width="0.9" marker-end="url(#ah)"/>')
    for i, (x0, y0) in enumerate(pts):
        colour = colors[i] if colors else sequential_color(i / max(n - 1, 1))
        f.parts.append(f'<circle cx="{f.px(x0):.1f}" cy="{f.py(y0):.1f}" r="3.5" fill="{colour}" stroke="#333" stroke-width="0.4"/>')
        if labels:
            f.parts.append(f'<text x="{f.px(x0) + 5:.1f}" y="{f.py(y0) - 4:.1f}" font-size="9">{html.escape(str(labels[i]))}</text>')
    return f.done()


def sequential_color(t: float) -> str:
    """Viridis-like ramp for t in [0, 1] (piecewise linear through five anchors)."""
    anchors = [(68, 1, 84), (59, 82, 139), (33, 145, 140), (94, 201, 98), (253, 231, 37)]
    t = min(max(float(t), 0.0), 1.0) * (len(anchors) - 1)
    i = min(int(t), len(anchors) - 2)
    a, b, u = anchors[i], anchors[i + 1], t - i
    return "#%02x%02x%02x" % tuple(int(round(a[k] + (b[k] - a[k]) * u)) for k in range(3))


def heatmap(matrix: Sequence[Sequence[float]], title: str = "", xlabel: str = "", ylabel: str = "",
            row_labels: Optional[Sequence[str]] = None, vmin: Optional[float] = None, vmax: Optional[float] = None,
            cell: int = 14) -> str:
    """Rows top to bottom, columns left to right, with a colour scale."""
    rows = [list(r) for r in matrix]
    nr, nc = len(rows), max((len(r) for r in rows), default=0)
    vals = _finite(v for r in rows for v in r) or [0.0, 1.0]
    lo, hi = (min(vals) if vmin is None else vmin), (max(vals) if vmax is None else vmax)
    span = (hi - lo) or 1.0
    left = 14 + (6 * max(len(str(s)) for s in row_labels) if row_labels else 26)
    top = 26 if title else 8
    w, h = left + nc * cell + 70, top + nr * cell + 34
    p = [f'<svg xmlns="http://www.w3.org/2000/svg" width="{w}" height="{h}" viewBox="0 0 {w} {h}" font-family="sans-serif" '
         f'font-size="10"><rect width="{w}" height="{h}" fill="white"/>']
    if title:
        p.append(f'<text x="{w / 2:.0f}" y="15" text-anchor="middle" font-size="12">{html.escape(title)}</text>')
    for i, r in enumerate(rows):
        label = str(row_labels[i]) if row_labels else (str(i) if nr <= 40 or i % 4 == 0 else "")
        p.append(f'<text x="{left - 4}" y="{top + i * cell + cell * 0.75:.1f}" text-anchor="end">{html.escape(label)}</text>')
        for j, v in enumerate(r):
            ok = v is not None and math.isfinite(float(v))
            colour = sequential_color((float(v) - lo) / span) if ok else "#dddddd"
            p.append(f'<rect x="{left + j * cell}" y="{top + i * cell}" width="{cell}" height="{cell}" fill="{colour}"/>')
    for j in range(0, nc, max(1, nc // 8)):
        p.append(f'<text x="{left + j * cell + cell / 2:.1f}" y="{top + nr * cell + 11}" text-anchor="middle">{j}</text>')
    bx = left + nc * cell + 12
    for k in range(40):
        p.append(f'<rect x="{bx}" y="{top + (39 - k) * nr * cell / 40:.1f}" width="10" height="{nr * cell / 40 + 0.5:.1f}" '
                 f'fill="{sequential_color(k / 39)}"/>')
    p.append(f'<text x="{bx + 14}" y="{top + 8}">{_fmt(hi)}</text><text x="{bx + 14}" y="{top + nr * cell}">{_fmt(lo)}</text>')
    if xlabel:
        p.append(f'<text x="{left + nc * cell / 2:.0f}" y="{h - 6}" text-anchor="middle">{html.escape(xlabel)}</text>')
    if ylabel:
        p.append(f'<text x="10" y="{top + nr * cell / 2:.0f}" text-anchor="middle" transform="rotate(-90 10 {top + nr * cell / 2:.0f})">'
                 f'{html.escape(ylabel)}</text>')
    return "".join(p) + "</svg>"


def bar_chart(values: dict[str, float], title: str = "", ylabel: str = "", colors: Optional[dict[str, str]] = None,
              w: int = 480, h: int = 280) -> str:
    names = list(values)
    vals = [float(values[n]) for n in names]
    f = _Frame([0, max(len(names), 1)], vals + [0.0], w, h, title, "", ylabel, x_ticks=False)
    bw = (w - f.l - f.r) / max(len(names), 1)
    for i, (n, v) in enumerate(zip(names, vals)):
        y0, y1 = f.py(0.0), f.py(v)
        colour = (colors or {}).get(n) or run_color(n)
        f.parts.append(f'<rect x="{f.l + i * bw + bw * 0.15:.1f}" y="{min(y0, y1):.1f}" width="{bw * 0.7:.1f}" height="{abs(y1 - y0):.1f}" '
                       f'fill="{colour}"/><text x="{f.l + (i + 0.5) * bw:.1f}" y="{h - f.b + 12}" text-anchor="middle">'
                       f'{html.escape(run_label(n, 12))}</text>')
    return f.done()
