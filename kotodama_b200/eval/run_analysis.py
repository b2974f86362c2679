"""Run-level analysis over JSONL metrics: endpoint summaries, training dynamics, geometric
health, run comparison, 2x2 factorial interaction and comparison against a reference run.

Function set and result keys follow ``src/eval/run_analysis.py`` of the reference
(``endpoint_summary :47``, ``training_dynamics :123``, ``geometric_health :410``,
``compare_runs :523``, ``factorial_analysis :591``, ``reference_comparison :722``).
"""
from __future__ import annotations

from typing import Any, Optional

from .core import extract_keys_matching, extract_series, get_nearest_step

StepData = dict[int, dict[str, float]]
DEFAULT_DYNAMICS_METRICS = ["train/loss", "geo/rankme_last"]
LANDMARK_PCTS = [0.10, 0.25, 0.50, 0.75, 0.90]
SLOPE_WINDOWS = [100, 500, 1000, 5000]
STABLE_RANK_PROJECTIONS = ["q_proj", "k_proj", "o_proj", "gate_proj", "down_proj"]


def _slope(pts: list[tuple[int, float]]) -> Optional[float]:
    n = len(pts)
    if n < 2:
        return None
    mx = sum(p[0] for p in pts) / n
    my = sum(p[1] for p in pts) / n
    den = sum((p[0] - mx) ** 2 for p in pts)
    return None if den < 1e-12 else sum((p[0] - mx) * (p[1] - my) for p in pts) / den


def _std(v: list[float]) -> float:
    if len(v) < 2:
        return 0.0
    m = sum(v) / len(v)
    return (sum((x - m) ** 2 for x in v) / (len(v) - 1)) ** 0.5


def _at(data: StepData, target: int, key: str, tolerance: int = 500) -> Optional[float]:
    series = {s: v for s, v in extract_series(data, key)}
    if not series:
        return None
    best = min(series, key=lambda s: abs(s - target))
    return series[best] if abs(best - target) <= tolerance else None


def endpoint_summary(data: StepData) -> dict[str, Any]:
    out: dict[str, Any] = {"max_step": max(data) if data else 0}
    loss = extract_series(data, "train/loss")
    if loss:
        lo = min(loss, key=lambda x: x[1])
        out.update(loss_initial=loss[0][1], loss_final=loss[-1][1], loss_min=lo[1], loss_min_step=lo[0])
    ppl = extract_series(data, "train/perplexity")
    if ppl:
        out["ppl_final"] = ppl[-1][1]
    tps = extract_series(data, "perf/tokens_per_sec")
    if tps:
        stable = tps[2:] if len(tps) > 2 else tps
        out["avg_tokens_per_sec"] = sum(v for _, v in stable) / len(stable)
    rk = extract_series(data, "geo/rankme_last")
    if rk:
        lo = min(rk, key=lambda x: x[1])
        out.update(rankme_initial=rk[0][1], rankme_min=lo[1], rankme_min_step=lo[0], rankme_final=rk[-1][1],
                   rankme_rebound_ratio=rk[-1][1] / max(lo[1], 1e-6))
    ww = extract_series(data, "geo/ww_alpha_mean")
    if ww:
        out.update(ww_alpha_initial=ww[0][1], ww_alpha_final=ww[-1][1])
    wh = extract_series(data, "geo/ww_alpha_healthy_frac")
    if wh:
        out["ww_healthy_frac_final"] = wh[-1][1]
    keys = extract_keys_matching(data, "geo/twonn_id/")
    if keys:
        def layer_of(k: str) -> int:
            try:
                return int(k.rsplit("_", 1)[1])
            except ValueError:
                return -1
        tw = extract_series(data, max(keys, key=layer_of))
        if tw:
            out["twonn_id_final"] = tw[-1][1]
    tok = extract_series(data, "data/tokens_consumed_B")
    if tok:
        out["tokens_B"] = tok[-1][1]
    return out


def _rolling(series: list[tuple[int, float]], window: int) -> list[tuple[int, float, float]]:
    out = []
    for i in range(len(series)):
        w = [v for s, v in series[max(0, i - window + 1): i + 1]]
        out.append((series[i][0], sum(w) / len(w), _std(w)))
    return out


def _plateaus(series: list[tuple[int, float]], window: int = 10, rel_tol: float = 1e-3) -> list[dict[str, Any]]:
    out, start = [], None
    for i in range(window, len(series)):
        seg = series[i - window: i + 1]
        sl = _slope(seg) or 0.0
        scale = abs(sum(v for _, v in seg) / len(seg)) + 1e-12
        span = max(seg[-1][0] - seg[0][0], 1)
        flat = abs(sl) * span / scale < rel_tol
        if flat and start is None:
            start = seg[0][0]
        if not flat and start is not None:
            out.append({"start_step": start, "end_step": series[i - 1][0]})
            start = None
    if start is not None:
        out.append({"start_step": start, "end_step": series[-1][0]})
    return out


def _jumps(series: list[tuple[int, float]], z: float = 4.0) -> list[dict[str, Any]]:
    diffs = [series[i + 1][1] - series[i][1] for i in range(len(series) - 1)]
    sd = _std(diffs)
    if sd == 0:
        return []
    m = sum(diffs) / len(diffs)
    return [{"step": series[i + 1][0], "delta": d, "z": (d - m) / sd} for i, d in enumerate(diffs) if abs(d - m) > z * sd]


def training_dynamics(data: StepData, metric_keys: Optional[list[str]] = None) -> dict[str, Any]:
    """Per metric: values at landmark fractions of the run, slopes over trailing windows, plateaus,
    jumps and slope sign changes."""
    out: dict[str, Any] = {}
    max_step = max(data) if data else 0
    for key in metric_keys or DEFAULT_DYNAMICS_METRICS:
        series = extract_series(data, key)
        if len(series) < 3:
            continue
        m: dict[str, Any] = {"n_points": len(series)}
        m["landmarks"] = {f"{int(p * 100)}%": _at(data, int(max_step * p), key, tolerance=max(500, max_step // 20))
                          for p in LANDMARK_PCTS}
        m["slopes"] = {}
        for w in SLOPE_WINDOWS:
            tail = [p for p in series if p[0] >= max_step - w]
            sl = _slope(tail)
            if sl is not None:
                m["slopes"][f"last_{w}"] = sl
        m["plateaus"] = _plateaus(series)
        m["jumps"] = _jumps(series)
        win = max(3, len(series) // 20)
        local = [(_slope(series[i - win: i + 1]) or 0.0, series[i][0]) for i in range(win, len(series))]
        m["slope_sign_changes"] = [s for (a, _), (b, s) in zip(local, local[1:]) if a * b < 0]
        roll = _rolling(series, win)
        m["final_rolling_mean"], m["final_rolling_std"] = roll[-1][1], roll[-1][2]
        out[key] = m
    return out


def _discover_layers(data: StepData) -> list[int]:
    layers = set()
    for k in extract_keys_matching(data, "geo/layer_"):
        try:
            layers.add(int(k.split("/")[1].split("_")[1]))
        except (IndexError, ValueError):
            pass
    return sorted(layers)


def geometric_health(data: StepData) -> dict[str, Any]:
    out: dict[str, Any] = {"layers": {}}
    for layer in _discover_layers(data):
        rec: dict[str, Any] = {}
        for proj in STABLE_RANK_PROJECTIONS:
            s = extract_series(data, f"geo/layer_{layer}/stable_rank_{proj}")
            if s:
                rec[f"stable_rank_{proj}"] = {"initial": s[0][1], "final": s[-1][1], "min": min(v for _, v in s)}
        for name in ("dead_units", "anisotropy", "attn_entropy_mean"):
            s = extract_series(data, f"geo/layer_{layer}/{name}")
            if s:
                rec[name] = {"initial": s[0][1], "final": s[-1][1]}
        out["layers"][layer] = rec
    alphas = {k.rsplit("_", 1)[1]: extract_series(data, k)[-1][1] for k in extract_keys_matching(data, "attnres/final_alpha/")
              if extract_series(data, k)}
    if alphas:
        out["attnres_final_alpha"] = alphas
    flags = []
    rk = extract_series(data, "geo/rankme_last")
    if rk and rk[-1][1] < 0.5 * max(v for _, v in rk):
        flags.append("rankme_collapse")
    for layer, rec in out["layers"].items():
        if rec.get("dead_units", {}).get("final", 0) > 0.1:
            flags.append(f"dead_units_layer_{layer}")
    out["flags"] = flags
    return out


def compare_runs(runs: dict[str, StepData], metric: str = "train/loss", at_steps: Optional[list[int]] = None
                 ) -> dict[str, Any]:
    summaries = {n: endpoint_summary(d) for n, d in runs.items()}
    common = min((s["max_step"] for s in summaries.values()), default=0)
    steps = at_steps or [int(common * p) for p in (0.25, 0.5, 0.75, 1.0)]
    table = {n: {s: _at(d, s, metric, tolerance=max(500, common // 20)) for s in steps} for n, d in runs.items()}
    final = {n: t[steps[-1]] for n, t in table.items() if t.get(steps[-1]) is not None}
    ranking = sorted(final, key=final.get)
    return {"summaries": summaries, "metric": metric, "steps": steps, "table": table, "ranking": ranking,
            "best": ranking[0] if ranking else None}


def factorial_analysis(runs: dict[tuple[int, int], StepData], metric: str = "train/loss", step: Optional[int] = None
                       ) -> dict[str, Any]:
    """2x2 design ``{(a, b): run}`` with a, b in {0, 1}: main effects and the interaction
    ``(y11 - y10) - (y01 - y00)`` of ``metric`` at ``step`` (default: last common step)."""
    need = [(0, 0), (0, 1), (1, 0), (1, 1)]
    if any(k not in runs for k in need):
        raise ValueError("factorial_analysis needs runs for (0,0), (0,1), (1,0), (1,1)")
    step = step if step is not None else min(max(d) for d in runs.values())
    y = {k: _at(runs[k], step, metric, tolerance=max(500, step // 20)) for k in need}
    if any(v is None for v in y.values()):
        return {"step": step, "values": y, "error": "metric missing for some cell"}
    a = ((y[(1, 0)] + y[(1, 1)]) - (y[(0, 0)] + y[(0, 1)])) / 2
    b = ((y[(0, 1)] + y[(1, 1)]) - (y[(0, 0)] + y[(1, 0)])) / 2
    inter = (y[(1, 1)] - y[(1, 0)]) - (y[(0, 1)] - y[(0, 0)])
    return {"step": step, "values": {f"{k[0]}{k[1]}": v for k, v in y.items()}, "main_effect_a": a,
            "main_effect_b": b, "interaction": inter}


def reference_comparison(run: StepData, reference: StepData, metrics: Optional[list[str]] = None) -> dict[str, Any]:
    """Differences run - reference at matched steps for the given metrics, plus the step at which the
    run first reaches the reference's final loss."""
    metrics = metrics or ["train/loss", "geo/rankme_last"]
    common = min(max(run) if run else 0, max(reference) if reference else 0)
    out: dict[str, Any] = {"common_step": common, "metrics": {}}
    for key in metrics:
        a, b = _at(run, common, key, tolerance=max(500, common // 20)), _at(reference, common, key, tolerance=max(500, common // 20))
        if a is not None and b is not None:
            out["metrics"][key] = {"run": a, "reference": b, "delta": a - b, "ratio": a / b if b else None}
    ref_loss = extract_series(reference, "train/loss")
    if ref_loss:
        target = ref_loss[-1][1]
        hit = next((s for s, v in extract_series(run, "train/loss") if v <= target), None)
        out["steps_to_reference_final_loss"] = hit
        if hit is not None and ref_loss[-1][0] > 0:
            out["speedup_vs_reference"] = ref_loss[-1][0] / max(hit, 1)
    return out
