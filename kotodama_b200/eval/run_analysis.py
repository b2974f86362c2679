"""Run-level analysis over JSONL metrics: endpoint summaries, training dynamics (multi-window slopes,
inflection points, rolling statistics, plateaus, jumps), geometric health (per-layer records, landmark
profiles, depth gradient), run comparison with direction-aware deltas, 2x2 factorial interaction with its
classification, and comparison against a reference run.  Pure functions over step-indexed dicts.

Function set and result keys follow ``src/eval/run_analysis.py`` of the reference
(``endpoint_summary :47``, ``training_dynamics :123``, ``geometric_health :410``,
``compare_runs :523``, ``factorial_analysis :591``, ``reference_comparison :722``).
"""
from __future__ import annotations

from typing import Any, Optional

from .core import extract_keys_matching, extract_series

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


def _jumps(series: list[tuple[int, float]], sigma_threshold: float = 3.0, warmup_frac: float = 0.05) -> list[dict[str, Any]]:
    """Step-over-step changes that stand out from the changes seen so far: after a warm-up (5 % of the points, at
    least 10) a change counts as a jump when it lies more than ``sigma_threshold`` standard deviations from the mean of
    all earlier changes (the reference's rule, ``src/eval/run_analysis.py:355-388``; running sums instead of its
    quadratic rescan).  The spread has a floor of 1e-9 of the series' scale, so rounding noise on a smooth curve is
    not a jump."""
    if len(series) < 20:
        return []
    vals = [v for _, v in series]
    deltas = [vals[i] - vals[i - 1] for i in range(1, len(vals))]
    floor = max(1e-10, 1e-9 * sum(abs(v) for v in vals) / len(vals))
    warm = max(10, int(len(series) * warmup_frac))
    out = []
    s1 = sum(deltas[:warm])
    s2 = sum(d * d for d in deltas[:warm])
    for i in range(warm, len(deltas)):
        mean = s1 / i
        sd = max(max(s2 / i - mean * mean, 0.0) ** 0.5, floor)
        dev = abs(deltas[i] - mean) / sd
        if dev > sigma_threshold:
            out.append({"step": series[i + 1][0], "delta": deltas[i], "sigma": round(dev, 2)})
        s1 += deltas[i]
        s2 += deltas[i] * deltas[i]
    return out


def _slope_at(series: list[tuple[int, float]], step: int, window: int) -> Optional[float]:
    """Least-squares slope over the points within ``window // 2`` steps on either side of ``step`` (at least three)."""
    half = window // 2
    pts = [p for p in series if step - half <= p[0] <= step + half]
    return _slope(pts) if len(pts) >= 3 else None


def _windowed_slopes(series: list[tuple[int, float]], window: int) -> list[tuple[int, float]]:
    """Slope of every consecutive stretch of ``window`` steps: [(stretch end, slope)]."""
    if len(series) < 3:
        return []
    out, lo = [], series[0][0]
    while lo < series[-1][0]:
        seg = [p for p in series if lo <= p[0] <= lo + window]
        sl = _slope(seg) if len(seg) >= 3 else None
        if sl is not None:
            out.append((seg[-1][0], sl))
        lo += window
    return out


def _sign_changes(series: list[tuple[int, float]], floor: float = 0.0) -> list[dict[str, Any]]:
    """Steps at which the series crosses zero; values within ``floor`` of zero (rounding noise) do not count."""
    big = [(st, v) for st, v in series if abs(v) > floor]
    return [{"step": s1, "from": a, "to": b} for (_, a), (s1, b) in zip(big, big[1:]) if a * b < 0]


def _percentile(v: list[float], q: float) -> float:
    w = sorted(v)
    at = q * (len(w) - 1)
    lo = int(at)
    return w[lo] + (w[min(lo + 1, len(w) - 1)] - w[lo]) * (at - lo)


def _rolling_stats(series: list[tuple[int, float]], window: int) -> list[dict[str, float]]:
    """Mean, sample spread and quartiles over consecutive stretches of ``window`` steps (stretches with fewer than two
    points are left out)."""
    out, lo = [], series[0][0] if series else 0
    while series and lo < max(series[-1][0], series[0][0] + 1):
        w = [v for st, v in series if lo <= st < lo + window]
        if len(w) >= 2:
            out.append({"step": lo + window, "step_center": lo + window // 2, "mean": sum(w) / len(w), "std": _std(w),
                        "p25": _percentile(w, 0.25), "p75": _percentile(w, 0.75), "n": len(w)})
        lo += window
    return out


def training_dynamics(data: StepData, metric_keys: Optional[list[str]] = None) -> dict[str, Any]:
    """Per metric: values and multi-window slopes at landmark fractions of the run, slopes over trailing
    windows, the second derivative's sign changes (inflection points), rolling statistics with a stability
    score (late spread / early spread), plateaus, jumps and slope sign changes."""
    out: dict[str, Any] = {}
    max_step = max(data) if data else 0
    for key in metric_keys or DEFAULT_DYNAMICS_METRICS:
        series = extract_series(data, key)
        if len(series) < 3:
            continue
        m: dict[str, Any] = {"n_points": len(series), "max_step": max_step}
        m["landmarks"] = {f"{int(p * 100)}%": _at(data, int(max_step * p), key, tolerance=max(500, max_step // 20))
                          for p in LANDMARK_PCTS}
        m["slopes_at_landmarks"] = {f"{int(p * 100)}%": {f"w{w}": _slope_at(series, int(max_step * p), w) for w in SLOPE_WINDOWS}
                                    for p in LANDMARK_PCTS}
        m["slopes"] = {}
        for w in SLOPE_WINDOWS:
            tail = [p for p in series if p[0] >= max_step - w]
            sl = _slope(tail)
            if sl is not None:
                m["slopes"][f"last_{w}"] = sl
        span = max(series[-1][0] - series[0][0], 1)
        coarse = _windowed_slopes(series, max(span // 20, 1))
        curv_floor = 1e-6 * max((abs(v) for _, v in coarse), default=0.0) / span
        m["inflection_points"] = _sign_changes(_windowed_slopes(coarse, max(span // 5, 1)), curv_floor) if len(coarse) >= 5 else []
        # 500-step stretches as in the reference once the run has at least ten of them, a twentieth of the run before
        roll_w = _rolling_stats(series, 500 if span >= 5000 else max(span // 20, 1))
        if roll_w:
            m["rolling_stats"] = roll_w
            n = len(roll_w)
            early = [r["std"] for r in roll_w[:max(n // 4, 1)] if r["std"] > 0]
            late = [r["std"] for r in roll_w[min(3 * n // 4, n - 1):] if r["std"] > 0]
            if early and late:
                m["stability_score"] = (sum(late) / len(late)) / max(sum(early) / len(early), 1e-10)
        m["plateaus"] = _plateaus(series)
        m["jumps"] = _jumps(series)
        win = max(3, len(series) // 20)
        local = [(_slope(series[i - win: i + 1]) or 0.0, series[i][0]) for i in range(win, len(series))]
        m["slope_sign_changes"] = [st for (a, _), (b, st) in zip(local, local[1:]) if a * b < 0]
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


GEO_LANDMARKS = {"early": 0.10, "quarter": 0.25, "mid": 0.50, "three_quarter": 0.75, "late": 0.90, "final": 1.0}
LAYER_METRICS = [f"stable_rank_{p}" for p in STABLE_RANK_PROJECTIONS] + ["attn_entropy_mean", "attn_entropy_std", "anisotropy", "dead_units"]


def geometric_health(data: StepData) -> dict[str, Any]:
    """Per-layer geometric record (initial / final / minimum of every per-layer metric), the same metrics as
    per-layer profiles at landmark fractions of the run (snapped to steps that carry geometric data), the
    depth gradient (first / middle / last sampled layer at the end of the run), the stability of RankMe
    (late spread / early spread), the routing weights of the final AttnRes call, and warning flags."""
    out: dict[str, Any] = {"layers": {}}
    layers = _discover_layers(data)
    for layer in layers:
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
    geo_steps = sorted(st for st in data if any(k.startswith("geo/layer_") for k in data[st]))
    if layers and geo_steps:
        max_step = max(data)
        marks = {n: min(geo_steps, key=lambda st: abs(st - int(max_step * p))) for n, p in GEO_LANDMARKS.items()}
        out["landmarks"] = marks
        out["profiles"] = {n: {"step": st, **{f"layer_{l}": {m: data[st].get(f"geo/layer_{l}/{m}") for m in LAYER_METRICS}
                                              for l in layers}} for n, st in marks.items()}
        if len(layers) >= 3:
            pick = {"first": layers[0], "mid": layers[len(layers) // 2], "last": layers[-1]}
            final = marks["final"]
            out["depth_gradient"] = {"layers": pick, **{m: {w: data[final].get(f"geo/layer_{l}/{m}") for w, l in pick.items()}
                                                        for m in ("attn_entropy_mean", "anisotropy", "stable_rank_q_proj")}}
    alphas = {k.rsplit("_", 1)[1]: extract_series(data, k)[-1][1] for k in extract_keys_matching(data, "attnres/final_alpha/")
              if extract_series(data, k)}
    if alphas:
        out["attnres_final_alpha"] = alphas
    flags = []
    rk = extract_series(data, "geo/rankme_last")
    if len(rk) >= 8:
        n = len(rk)                                  # first quarter against last quarter, cut as the reference cuts them
        out["rankme_stability"] = _std([v for _, v in rk[3 * n // 4:]]) / max(_std([v for _, v in rk[:n // 4]]), 1e-10)
    if rk and rk[-1][1] < 0.5 * max(v for _, v in rk):
        flags.append("rankme_collapse")
    for layer, rec in out["layers"].items():
        if rec.get("dead_units", {}).get("final", 0) > 0.1:
            flags.append(f"dead_units_layer_{layer}")
        ent = rec.get("attn_entropy_mean", {})
        if ent and ent.get("initial") and ent["final"] < 0.25 * ent["initial"]:
            flags.append(f"attention_collapse_layer_{layer}")
    out["flags"] = flags
    return out


LOWER_IS_BETTER = {"loss_final", "loss_min", "ppl_final", "ww_alpha_final"}
COMPARISON_KEYS = ["loss_final", "loss_min", "ppl_final", "rankme_final", "rankme_min", "rankme_rebound_ratio", "ww_alpha_final",
                   "ww_healthy_frac_final", "twonn_id_final", "avg_tokens_per_sec", "tokens_B"]


def compare_runs(runs: dict[str, StepData], metric: str = "train/loss", at_steps: Optional[list[int]] = None
                 ) -> dict[str, Any]:
    """Endpoint summaries side by side, ``metric`` at matched steps, a ranking by its last matched value, and
    for every run after the first the deltas of the endpoint figures against the first run, each marked
    better / worse according to the figure's direction (loss down, RankMe up, ...)."""
    summaries = {n: endpoint_summary(d) for n, d in runs.items()}
    common = min((s["max_step"] for s in summaries.values()), default=0)
    steps = at_steps or [int(common * p) for p in (0.25, 0.5, 0.75, 1.0)]
    table = {n: {s: _at(d, s, metric, tolerance=max(500, common // 20)) for s in steps} for n, d in runs.items()}
    final = {n: t[steps[-1]] for n, t in table.items() if t.get(steps[-1]) is not None}
    ranking = sorted(final, key=final.get)
    names = list(runs)
    deltas: dict[str, dict[str, Any]] = {}
    for n in names[1:]:
        row = {}
        for k in COMPARISON_KEYS:
            a, b = summaries[names[0]].get(k), summaries[n].get(k)
            if isinstance(a, (int, float)) and isinstance(b, (int, float)):
                d = b - a
                better = d < 0 if k in LOWER_IS_BETTER else d > 0
                row[k] = {"delta": d, "relative": d / abs(a) if a else None,
                          "verdict": "same" if d == 0 else ("better" if better else "worse")}
        deltas[n] = row
    best_per_metric = {}
    for k in COMPARISON_KEYS:                       # which run wins each endpoint figure, by the figure's direction
        have = {n: sm[k] for n, sm in summaries.items() if isinstance(sm.get(k), (int, float))}
        if have:
            best_per_metric[k] = (min if k in LOWER_IS_BETTER else max)(have, key=have.get)
    return {"summaries": summaries, "metric": metric, "steps": steps, "table": table, "ranking": ranking,
            "best": ranking[0] if ranking else None, "best_per_metric": best_per_metric,
            "baseline": names[0] if names else None, "deltas": deltas}


def _factorial_cell(y: dict[tuple[int, int], float]) -> dict[str, Any]:
    a = ((y[(1, 0)] + y[(1, 1)]) - (y[(0, 0)] + y[(0, 1)])) / 2
    b = ((y[(0, 1)] + y[(1, 1)]) - (y[(0, 0)] + y[(1, 0)])) / 2
    inter = (y[(1, 1)] - y[(1, 0)]) - (y[(0, 1)] - y[(0, 0)])
    additive = y[(0, 0)] + (y[(1, 0)] - y[(0, 0)]) + (y[(0, 1)] - y[(0, 0)])         # what "no interaction" predicts for both
    scale = max(abs(y[(1, 0)] - y[(0, 0)]), abs(y[(0, 1)] - y[(0, 0)]), 1e-12)
    rel = inter / scale
    kind = "additive" if abs(rel) < 0.1 else ("reinforcing" if (inter < 0) == (a + b < 0) else "offsetting")
    # the reference's label: by the sign of the interaction, additive below 5 % of the summed main effects
    sign = "additive" if abs(inter) < 0.05 * abs(a + b) else ("super-additive" if inter > 0 else "sub-additive")
    return {"values": {f"{k[0]}{k[1]}": v for k, v in y.items()}, "main_effect_a": a, "main_effect_b": b, "interaction": inter,
            "additive_prediction": additive, "relative_interaction": rel, "classification": kind, "additivity": sign}


def factorial_analysis(runs: dict[tuple[int, int], StepData], metric: str = "train/loss", step: Optional[int] = None,
                       extra_metrics: Optional[list[str]] = None, all_metrics: bool = False) -> dict[str, Any]:
    """2x2 design ``{(a, b): run}`` with a, b in {0, 1}: main effects and the interaction
    ``(y11 - y10) - (y01 - y00)`` of ``metric`` at ``step`` (default: last common step), what a purely
    additive model predicts for the cell with both factors, the interaction relative to the larger
    single-factor effect and its classification (additive below 10 %; reinforcing when it pushes the same
    way as the main effects, offsetting otherwise; ``additivity`` is the reference's sign-based label).
    ``extra_metrics``: the same for further metrics; ``all_metrics``: for every numeric metric that all four runs
    logged at that step, as the reference's ``factorial_analysis`` reports."""
    need = [(0, 0), (0, 1), (1, 0), (1, 1)]
    if any(k not in runs for k in need):
        raise ValueError("factorial_analysis needs runs for (0,0), (0,1), (1,0), (1,1)")
    step = step if step is not None else min(max(d) for d in runs.values())
    tol = max(500, step // 20)
    y = {k: _at(runs[k], step, metric, tolerance=tol) for k in need}
    if any(v is None for v in y.values()):
        return {"step": step, "values": y, "error": "metric missing for some cell"}
    out = {"step": step, "metric": metric, **_factorial_cell(y)}
    others = {}
    keys = list(extra_metrics or [])
    if all_metrics:
        found: set[str] = set()
        for k in need:
            near = min(runs[k], key=lambda st: abs(st - step)) if runs[k] else None
            if near is not None:
                found.update(name for name, v in runs[k][near].items() if isinstance(v, (int, float)) and not isinstance(v, bool))
        keys += sorted(found - set(keys) - {metric})
    for key in keys:
        ys = {k: _at(runs[k], step, key, tolerance=tol) for k in need}
        if all(v is not None for v in ys.values()):
            others[key] = _factorial_cell(ys)
    if others:
        out["other_metrics"] = others
    return out


def summary_comparison(run: StepData, reference: dict[str, Any], threshold_pct: float = 10.0) -> dict[str, Any]:
    """The run's endpoint summary against a reference *summary* (the output of `endpoint_summary` for another run, or
    hand-written target values): per shared numeric figure the delta and the change in per cent, and the figures that
    moved by more than ``threshold_pct`` (the reference's ``reference_comparison``, ``src/eval/run_analysis.py:722-777``)."""
    current = endpoint_summary(run)
    comparisons: dict[str, dict[str, Any]] = {}
    flagged: list[dict[str, Any]] = []
    for key, ref_val in reference.items():
        cur = current.get(key)
        if isinstance(ref_val, bool) or not isinstance(ref_val, (int, float)) or cur is None:
            continue
        delta = cur - ref_val
        pct = delta / abs(ref_val) * 100 if abs(ref_val) > 1e-10 else 0.0
        comparisons[key] = {"reference": ref_val, "current": cur, "delta": delta, "pct_change": round(pct, 2)}
        if abs(pct) > threshold_pct:
            flagged.append({"metric": key, **comparisons[key]})
    return {"comparisons": comparisons, "flagged": flagged, "threshold_pct": threshold_pct}


def reference_comparison(run: StepData, reference: Any, metrics: Optional[list[str]] = None,
                         threshold_pct: float = 10.0) -> dict[str, Any]:
    """Differences run - reference at matched steps for the given metrics, plus the step at which the
    run first reaches the reference's final loss.  When ``reference`` is a summary (figure name -> value) instead of
    step-indexed metrics, the endpoint summaries are compared (`summary_comparison`)."""
    if reference and all(isinstance(k, str) for k in reference):
        return summary_comparison(run, reference, threshold_pct)
    metrics = metrics or ["train/loss", "geo/rankme_last"]
    common = min(max(run) if run else 0, max(reference) if reference else 0)
    out: dict[str, Any] = {"common_step": common, "metrics": {}}
    for key in metrics:
        a, b = _at(run, common, key, tolerance=max(500, common // 20)), _at(reference, common, key, tolerance=max(500, common // 20))
        if a is not None and b is not None:
            out["metrics"][key] = {"run": a, "reference": b, "delta": a - b, "ratio": a / b if b else None}
    # the same deltas along the run: does the gap open early or late?
    out["landmarks"] = {}
    for p in LANDMARK_PCTS:
        st = int(common * p)
        row = {}
        for key in metrics:
            a, b = _at(run, st, key, tolerance=max(500, common // 20)), _at(reference, st, key, tolerance=max(500, common // 20))
            if a is not None and b is not None:
                row[key] = a - b
        out["landmarks"][f"{int(p * 100)}%"] = {"step": st, "delta": row}
    ref_loss = extract_series(reference, "train/loss")
    if ref_loss:
        target = ref_loss[-1][1]
        hit = next((s for s, v in extract_series(run, "train/loss") if v <= target), None)
        out["steps_to_reference_final_loss"] = hit
        if hit is not None and ref_loss[-1][0] > 0:
            out["speedup_vs_reference"] = ref_loss[-1][0] / max(hit, 1)
    return out
