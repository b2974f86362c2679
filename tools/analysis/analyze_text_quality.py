#!/usr/bin/env python
"""Text-quality metrics of generated samples (track 4).  Five metric families, the ones of the
reference's ``scripts/analysis/analyze_text_quality.py`` (its ``LexicalMetrics``, ``CoherenceMetrics``,
``StructuralMetrics``, ``RepetitionMetrics`` and ``CreativityMetrics``), computed here with regular
expressions and closed word lists only - no NLTK / tagger models, so it runs offline:

  lexical      type/token ratios of the first 50/100/200/500 words and of the whole sample, moving-average
               type/token ratios, hapax ratio, Yule's K, Honore's R,
               part-of-speech shares from closed classes + suffix rules, sentence-length statistics,
               punctuation variety
  coherence    cosine similarity of consecutive sentences (topic drift: mean, spread, slope), novelty
               curve (new word types per window: mean, spread, slope, last vs first window), entity
               count and introduction rate, pronoun-to-noun density
  structure    clause-depth estimate, discourse markers, sentence types and their entropy, register
               consistency (spread of per-sentence formality)
  repetition   onset of the first repeated 5-gram, size of repeated units, unique n-gram ratios
               (1/2/3/5/8), novel tokens after the onset, terminal loop period
  creativity   specificity (numbers, names, dates), temporal / dialogue markers, quotes, density of
               unsupported-claim patterns, distance of a sample from the other answers to its prompt

One ``--input`` gives per-prompt and overall figures; several give a per-run profile table and, per
run, the metrics on which it differs most from the others (z-score over runs).

    python tools/analysis/analyze_text_quality.py --input analysis/runA/generations.json
    python tools/analysis/analyze_text_quality.py --input analysis/runA/generations.json analysis/runB/generations.json \\
        --output analysis/text_quality --csv
"""
from __future__ import annotations

import argparse
import csv
import json
import math
import re
from collections import Counter
from pathlib import Path
from statistics import mean, pstdev
from typing import Any, Iterable, Sequence

from _common import write_json

WORD = re.compile(r"[A-Za-z0-9]+(?:'[A-Za-z]+)?")
SENT = re.compile(r"(?<=[.!?])[\"')\]]*\s+")

PRONOUNS = set("i you he she it we they me him her us them my your his its our their mine yours hers ours theirs this that "
               "these those who whom whose which myself yourself himself herself itself ourselves themselves".split())
DETERMINERS = set("a an the some any each every no either neither".split())
PREPOSITIONS = set("of in on at by for with about against between into through during before after above below to from up down "
                   "over under again further within without across behind beyond near among".split())
AUXILIARIES = set("is are was were be been being am do does did have has had will would shall should can could may might must".split())
CONJUNCTIONS = set("and or but nor so yet for".split())
SUBORDINATORS = set("because although though while whereas when whenever if unless until since that which who whom whose where "
                    "after before as once than whether".split())
DISCOURSE = ["however", "therefore", "moreover", "furthermore", "nevertheless", "meanwhile", "consequently", "thus", "hence",
             "instead", "otherwise", "for example", "for instance", "in addition", "in contrast", "on the other hand", "as a result",
             "in fact", "of course", "in conclusion", "first", "second", "finally", "then", "next", "also", "besides", "still"]
TEMPORAL = ["yesterday", "today", "tomorrow", "tonight", "now", "then", "later", "earlier", "soon", "once", "never", "always",
            "before", "after", "during", "while", "until", "since", "ago", "morning", "evening", "night", "week", "month", "year",
            "century", "monday", "tuesday", "wednesday", "thursday", "friday", "saturday", "sunday", "january", "february", "march",
            "april", "june", "july", "august", "september", "october", "november", "december"]
DIALOGUE = ["said", "asked", "replied", "answered", "whispered", "shouted", "told", "cried", "muttered", "exclaimed", "says", "asks"]
IMPERATIVE_STARTS = set("let please do don't take make go come look see try keep stop remember consider note imagine think tell give "
                        "put use find add remove check open close turn run".split())
INFORMAL = set("gonna wanna gotta kinda sorta yeah yep nope ok okay hey wow oh ah um uh lol stuff thing things really very just "
               "like totally pretty".split())
CLAIM_PATTERNS = [r"according to [A-Z]", r"\bstud(?:y|ies) (?:show|shows|found|suggest)", r"\bresearch(?:ers)? (?:show|shows|found|suggest)",
                  r"\bexperts? (?:say|says|agree|believe)", r"\bit is (?:well )?known that", r"\bscientists? (?:say|says|found|believe)",
                  r"\b\d{1,3}(?:\.\d+)? ?(?:%|percent)", r"\bin (?:1[5-9]|20)\d\d\b", r"\b(?:Dr|Prof|Professor)\.? [A-Z][a-z]+",
                  r"\bpublished in\b", r"\ba (?:recent )?(?:survey|report|poll)\b"]
CLAIM_RE = [re.compile(p) for p in CLAIM_PATTERNS]


# ----------------------------------------------------------------------------- helpers
def words(text: str) -> list[str]:
    return [w.lower() for w in WORD.findall(text)]


def sentences(text: str) -> list[str]:
    return [s.strip() for s in SENT.split(text.strip()) if s.strip()]


def safe_div(a: float, b: float, default: float = 0.0) -> float:
    return a / b if b else default


def spread(xs: Sequence[float]) -> float:
    return pstdev(xs) if len(xs) > 1 else 0.0


def slope(ys: Sequence[float]) -> float:
    """Least-squares slope of ``ys`` against 0, 1, 2, ..."""
    n = len(ys)
    if n < 2:
        return 0.0
    mx, my = (n - 1) / 2, mean(ys)
    num = sum((i - mx) * (y - my) for i, y in enumerate(ys))
    den = sum((i - mx) ** 2 for i in range(n))
    return num / den


def entropy(counts: Iterable[float]) -> float:
    c = [x for x in counts if x > 0]
    tot = sum(c)
    return -sum(x / tot * math.log2(x / tot) for x in c) if tot else 0.0


def ngrams(ws: Sequence[str], n: int) -> list[tuple]:
    return [tuple(ws[i:i + n]) for i in range(len(ws) - n + 1)]


def cosine(a: Counter, b: Counter) -> float:
    dot = sum(v * b.get(k, 0) for k, v in a.items())
    na, nb = math.sqrt(sum(v * v for v in a.values())), math.sqrt(sum(v * v for v in b.values()))
    return safe_div(dot, na * nb)


def content(ws: Iterable[str]) -> list[str]:
    closed = PRONOUNS | DETERMINERS | PREPOSITIONS | AUXILIARIES | CONJUNCTIONS | SUBORDINATORS
    return [w for w in ws if w not in closed and len(w) > 2]


def guess_pos(w: str) -> str:
    """Coarse part of speech from closed classes and suffixes; good enough for ratios over a sample."""
    if w in PRONOUNS:
        return "pron"
    if w in DETERMINERS or w in PREPOSITIONS or w in CONJUNCTIONS or w in SUBORDINATORS:
        return "func"
    if w in AUXILIARIES:
        return "verb"
    if w.endswith("ly") and len(w) > 4:
        return "adv"
    if w.endswith(("ing", "ed", "ize", "ise", "ify", "ate")) and len(w) > 4:
        return "verb"
    if w.endswith(("ous", "ful", "ive", "able", "ible", "al", "ic", "ish", "less", "ary")) and len(w) > 4:
        return "adj"
    if w.isdigit():
        return "num"
    return "noun"


# ----------------------------------------------------------------------------- the five families
def head_ttr(ws: Sequence[str], window: int) -> float:
    """Type/token ratio of the first ``window`` words (the reference's ``compute_ttr``): comparable across samples of
    different length because every sample is cut to the same number of words."""
    head = ws[:window]
    return len(set(head)) / len(head) if head else 0.0


def windowed_ttr(ws: Sequence[str], window: int) -> float:
    """Moving-average type/token ratio: the mean over windows of ``window`` words, half a window apart."""
    if not ws:
        return 0.0
    if len(ws) <= window:
        return len(set(ws)) / len(ws)
    step = max(1, window // 2)
    vals = [len(set(ws[i:i + window])) / window for i in range(0, len(ws) - window + 1, step)]
    return mean(vals)


def yules_k(ws: Sequence[str]) -> float:
    """10^4 (sum_i i^2 V_i - N) / N^2 with V_i the number of types occurring i times; lower = richer."""
    n = len(ws)
    if n < 2:
        return 0.0
    spectrum = Counter(Counter(ws).values())
    return max(1e4 * (sum(i * i * v for i, v in spectrum.items()) - n) / (n * n), 0.0)


def honores_r(ws: Sequence[str]) -> float:
    """100 log(N + 1) / (1 - V1 / V): rewards types used exactly once (N + 1 as in the reference's ``compute_honores_r``)."""
    n, c = len(ws), Counter(ws)
    v, v1 = len(c), sum(1 for x in c.values() if x == 1)
    if n < 2 or v == 0 or v1 == v:
        return 0.0
    return 100 * math.log(n + 1) / (1 - v1 / v)


def lexical(text: str) -> dict[str, float]:
    ws, ss = words(text), sentences(text)
    c = Counter(ws)
    pos = Counter(guess_pos(w) for w in ws)
    slen = [len(words(s)) for s in ss if words(s)] or [0]
    punct = [ch for ch in text if ch in ".,;:!?-—()[]\"'…"]
    n = max(len(ws), 1)
    return {"tokens": len(ws), "ttr_50": head_ttr(ws, 50), "ttr_100": head_ttr(ws, 100), "ttr_200": head_ttr(ws, 200),
            "ttr_500": head_ttr(ws, 500), "ttr_all": safe_div(len(c), len(ws)),
            "mattr_50": windowed_ttr(ws, 50), "mattr_100": windowed_ttr(ws, 100),
            "hapax_ratio": safe_div(sum(1 for v in c.values() if v == 1), len(c)), "yules_k": yules_k(ws), "honores_r": honores_r(ws),
            "pos_noun_ratio": pos["noun"] / n, "pos_verb_ratio": pos["verb"] / n, "pos_adj_ratio": pos["adj"] / n,
            "pos_adv_ratio": pos["adv"] / n, "pos_pronoun_ratio": pos["pron"] / n,
            "sent_len_mean": mean(slen), "sent_len_std": spread(slen), "sent_len_min": min(slen), "sent_len_max": max(slen),
            "sent_count": len(ss), "punct_types": len(set(punct)), "punct_ratio": safe_div(len(punct), len(text)),
            "mean_word_len": mean(map(len, ws)) if ws else 0.0}


def coherence(text: str) -> dict[str, float]:
    ws, ss = words(text), sentences(text)
    bags = [Counter(content(words(s))) for s in ss]
    bags = [b for b in bags if b]
    sims = [cosine(a, b) for a, b in zip(bags, bags[1:])]
    # novelty curve: share of word types in each 50-token window that have not occurred before
    seen: set[str] = set()
    novelty = []
    for i in range(0, len(ws), 50):
        win = ws[i:i + 50]
        if len(win) < 10:
            break
        types = set(win)
        novelty.append(len(types - seen) / len(types))
        seen |= types
    ents = re.findall(r"(?<![.!?]\s)(?<!^)(?<![\"'(])\b[A-Z][a-z]{2,}(?:\s[A-Z][a-z]{2,})*", text)
    pos = Counter(guess_pos(w) for w in ws)
    return {"topic_similarity_mean": mean(sims) if sims else 0.0, "topic_drift_mean": 1 - mean(sims) if sims else 0.0,
            "topic_drift_std": spread(sims), "topic_drift_trend": -slope(sims),
            "novelty_mean": mean(novelty) if novelty else 0.0, "novelty_std": spread(novelty), "novelty_trend": slope(novelty),
            "novelty_final_vs_initial": safe_div(novelty[-1], novelty[0]) if novelty else 0.0,
            "entity_count": len(set(ents)), "entity_intro_rate": 100 * safe_div(len(set(ents)), len(ws)),
            "referential_density": safe_div(pos["pron"], pos["noun"])}


def sentence_type(s: str) -> str:
    t = s.rstrip("\"')] ")
    first = (words(s) or [""])[0]
    if t.endswith("?"):
        return "interrogative"
    if t.endswith("!"):
        return "exclamatory"
    if first in IMPERATIVE_STARTS:
        return "imperative"
    return "declarative"


def clause_depth(s: str) -> int:
    """1 + subordinators + paired commas / brackets: a rough count of nested or attached clauses."""
    ws = words(s)
    sub = sum(1 for w in ws if w in SUBORDINATORS)
    return 1 + sub + s.count(",") // 2 + s.count("(") + s.count(";")


def formality(s: str) -> float:
    ws = words(s)
    if not ws:
        return 0.0
    long_words = sum(1 for w in ws if len(w) >= 7) / len(ws)
    informal = sum(1 for w in ws if w in INFORMAL or "'" in w) / len(ws)
    return long_words - informal


def structural(text: str) -> dict[str, float]:
    ws, ss = words(text), sentences(text)
    low = " " + " ".join(ws) + " "
    markers = sum(low.count(" " + m + " ") for m in DISCOURSE)
    kinds = Counter(sentence_type(s) for s in ss)
    depth = [clause_depth(s) for s in ss] or [0]
    form = [formality(s) for s in ss if words(s)]
    n = max(len(ss), 1)
    return {"clause_depth_mean": mean(depth), "clause_depth_std": spread(depth), "discourse_marker_count": markers,
            "discourse_marker_density": 100 * safe_div(markers, len(ws)), "structural_variety_entropy": entropy(kinds.values()),
            "pct_declarative": kinds["declarative"] / n, "pct_interrogative": kinds["interrogative"] / n,
            "pct_exclamatory": kinds["exclamatory"] / n, "pct_imperative": kinds["imperative"] / n,
            "register_consistency_mean": mean(form) if form else 0.0, "register_consistency_std": spread(form)}


def loop_period(ws: Sequence[str], min_reps: int = 3) -> int:
    """Smallest period p such that the text ends in >= min_reps copies of a p-word unit (0 = none)."""
    for p in range(1, min(64, len(ws) // min_reps) + 1):
        unit = ws[-p:]
        if all(ws[len(ws) - (r + 1) * p:len(ws) - r * p] == unit for r in range(min_reps)):
            return p
    return 0


def repetition(text: str) -> dict[str, float]:
    ws = words(text)
    out: dict[str, float] = {}
    for n in (1, 2, 3, 5, 8):
        g = ngrams(ws, n)
        out[f"unique_{n}gram_ratio"] = safe_div(len(set(g)), len(g), 1.0)
    # onset: position (in tokens) of the first 5-gram that has been seen before
    seen: dict[tuple, int] = {}
    onset = -1
    for i, g in enumerate(ngrams(ws, 5)):
        if g in seen:
            onset = i
            break
        seen[g] = i
    out["repetition_onset_5gram"] = onset
    # repeated units: maximal runs of consecutive positions whose 5-gram is a repeat
    c5 = Counter(ngrams(ws, 5))
    runs, cur = [], 0
    for g in ngrams(ws, 5):
        if c5[g] > 1:
            cur += 1
        elif cur:
            runs.append(cur + 4)
            cur = 0
    if cur:
        runs.append(cur + 4)
    out["repetition_unit_size_mean"] = mean(runs) if runs else 0.0
    out["repetition_unit_size_max"] = max(runs) if runs else 0
    if onset >= 0:
        before = set(ws[:onset])
        after = ws[onset:]
        novel = sum(1 for w in set(after) if w not in before)
        out["post_rep_novel_tokens"] = novel
        out["post_rep_novel_ratio"] = safe_div(novel, len(set(after)))
    else:
        out["post_rep_novel_tokens"] = 0
        out["post_rep_novel_ratio"] = 1.0
    out["loop_period"] = loop_period(ws)
    return out


def creativity(text: str, siblings: Sequence[Counter] = ()) -> dict[str, float]:
    ws = words(text)
    n = max(len(ws), 1)
    numbers = len(re.findall(r"\b\d[\d,.]*\b", text))
    names = len(re.findall(r"(?<![.!?]\s)(?<!^)\b[A-Z][a-z]{2,}", text))
    dates = len(re.findall(r"\b(?:1[0-9]|20)\d\d\b", text))
    temporal = sum(1 for w in ws if w in TEMPORAL)
    dialogue = sum(1 for w in ws if w in DIALOGUE)
    quotes = len(re.findall(r"\"[^\"]{2,}\"|“[^”]{2,}”", text))
    claims = sum(len(r.findall(text)) for r in CLAIM_RE)
    mine = Counter(content(ws))
    if siblings:
        centre: Counter = Counter()
        for s in siblings:
            centre.update(s)
        unexpected = 1 - cosine(mine, centre)
    else:
        unexpected = 0.0
    return {"specificity_score": 100 * (numbers + names + 2 * dates) / n, "temporal_marker_count": temporal,
            "temporal_marker_density": 100 * temporal / n, "dialogue_marker_count": dialogue, "dialogue_marker_density": 100 * dialogue / n,
            "quote_count": quotes, "fabrication_density": 100 * claims / n, "topical_unexpectedness": unexpected,
            "ends_terminated": 1.0 if text.rstrip()[-1:] in ".!?\"'”" else 0.0}


FAMILIES = ("lexical", "coherence", "structural", "repetition", "creativity")


def analyse(text: str, siblings: Sequence[Counter] = ()) -> dict[str, Any]:
    if not words(text):
        return {"empty": True}
    return {"lexical": lexical(text), "coherence": coherence(text), "structural": structural(text),
            "repetition": repetition(text), "creativity": creativity(text, siblings)}


def flatten(row: dict[str, Any]) -> dict[str, float]:
    return {f"{fam}.{k}": float(v) for fam in FAMILIES for k, v in row[fam].items()}


def aggregate(rows: list[dict[str, Any]]) -> dict[str, Any]:
    rows = [r for r in rows if not r.get("empty")]
    out: dict[str, Any] = {"n": len(rows)}
    if not rows:
        return out
    for fam in FAMILIES:
        out[fam] = {k: mean(float(r[fam][k]) for r in rows) for k in rows[0][fam]}
    out["loop_rate"] = mean(1.0 if r["repetition"]["loop_period"] > 0 else 0.0 for r in rows)
    out["repeat_rate"] = mean(1.0 if r["repetition"]["repetition_onset_5gram"] >= 0 else 0.0 for r in rows)
    return out


# ----------------------------------------------------------------------------- runs, profiles, reports
def analyse_file(path: Path) -> dict[str, Any]:
    data = json.loads(path.read_text())
    gens = data["generations"] if isinstance(data, dict) else data
    per_prompt, everything = [], []
    for g in gens:
        samples = g["samples"] if "samples" in g else [g.get("text", "")]
        bags = [Counter(content(words(s))) for s in samples]
        rows = [analyse(s, bags[:i] + bags[i + 1:]) for i, s in enumerate(samples)]
        everything += rows
        per_prompt.append({"prompt": g.get("prompt", ""), "metrics": aggregate(rows)})
    run = (data.get("run") if isinstance(data, dict) else None) or path.parent.name
    return {"run": run, "source": str(path), "overall": aggregate(everything), "per_prompt": per_prompt}


def profile(result: dict[str, Any]) -> dict[str, float]:
    o = result["overall"]
    flat = {f"{fam}.{k}": v for fam in FAMILIES for k, v in o.get(fam, {}).items()}
    flat["loop_rate"], flat["repeat_rate"] = o.get("loop_rate", 0.0), o.get("repeat_rate", 0.0)
    return flat


def most_distinctive(profiles: dict[str, dict[str, float]], top: int = 8) -> dict[str, list[tuple[str, float, float]]]:
    """Per run: the metrics whose value lies furthest (in standard deviations over runs) from the mean of all runs."""
    out: dict[str, list] = {}
    keys = sorted(set().union(*[set(p) for p in profiles.values()]))
    stats = {}
    for k in keys:
        vals = [p.get(k, 0.0) for p in profiles.values()]
        stats[k] = (mean(vals), spread(vals))
    for run, p in profiles.items():
        z = [(k, safe_div(p.get(k, 0.0) - stats[k][0], stats[k][1]), p.get(k, 0.0)) for k in keys if stats[k][1] > 0]
        out[run] = sorted(z, key=lambda t: -abs(t[1]))[:top]
    return out


HEADLINE = ["lexical.ttr_100", "lexical.yules_k", "lexical.sent_len_mean", "coherence.topic_drift_mean", "coherence.novelty_mean",
            "structural.clause_depth_mean", "structural.structural_variety_entropy", "repetition.unique_3gram_ratio",
            "repetition.repetition_unit_size_max", "repeat_rate", "loop_rate", "creativity.specificity_score",
            "creativity.fabrication_density"]


def comparison_table(profiles: dict[str, dict[str, float]], keys: Sequence[str] = HEADLINE) -> str:
    runs = list(profiles)
    w = max(len(k) for k in keys) + 2
    lines = [" " * w + "".join(f"{r[:14]:>16s}" for r in runs)]
    for k in keys:
        lines.append(f"{k:<{w}s}" + "".join(f"{profiles[r].get(k, float('nan')):16.4f}" for r in runs))
    return "\n".join(lines)


def full_report(results: list[dict[str, Any]]) -> str:
    out = []
    for res in results:
        o = res["overall"]
        out.append(f"== {res['run']}  ({o.get('n', 0)} samples, {res['source']})")
        for fam in FAMILIES:
            out.append(f"  [{fam}]")
            for k, v in o.get(fam, {}).items():
                out.append(f"    {k:34s} {v:12.4f}")
        out.append(f"  repeat_rate {o.get('repeat_rate', 0.0):.3f}   loop_rate {o.get('loop_rate', 0.0):.3f}")
    return "\n".join(out)


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True, nargs="+", help="generations.json of eval_generate / eval_via_server (one per run)")
    ap.add_argument("--output", default=None, help="output file (one input) or directory (several)")
    ap.add_argument("--csv", action="store_true", help="also write the per-run profiles as CSV")
    ap.add_argument("--full", action="store_true", help="print every metric, not only the headline table")
    a = ap.parse_args()
    results = [analyse_file(Path(p)) for p in a.input]
    profiles = {r["run"]: profile(r) for r in results}
    if len(results) == 1:
        dst = Path(a.output) if a.output else Path(a.input[0]).with_name("text_quality.json")
        write_json(dst, results[0])
        out_dir = dst.parent
    else:
        out_dir = Path(a.output) if a.output else Path("analysis/text_quality")
        out_dir.mkdir(parents=True, exist_ok=True)
        distinct = most_distinctive(profiles)
        write_json(out_dir / "text_quality_comparison.json",
                   {"runs": results, "profiles": profiles,
                    "most_distinctive": {r: [{"metric": k, "z": z, "value": v} for k, z, v in rows] for r, rows in distinct.items()}})
        dst = out_dir / "text_quality_comparison.json"
        for run, rows in distinct.items():
            print(f"{run}: " + ", ".join(f"{k} ({z:+.1f} sd)" for k, z, _ in rows[:4]))
    if a.csv:
        keys = sorted(set().union(*[set(p) for p in profiles.values()]))
        with open(out_dir / "text_quality_profiles.csv", "w", newline="") as fh:
            wr = csv.writer(fh)
            wr.writerow(["run"] + keys)
            for run, p in profiles.items():
                wr.writerow([run] + [f"{p.get(k, 0.0):.6g}" for k in keys])
    print(full_report(results) if a.full else comparison_table(profiles))
    print(f"{sum(r['overall'].get('n', 0) for r in results)} samples -> {dst}")


if __name__ == "__main__":
    main()
