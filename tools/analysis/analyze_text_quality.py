#!/usr/bin/env python
"""Text-quality metrics of generated samples (track 4), five layers as in the reference's
``scripts/analysis/analyze_text_quality.py``, computed without external NLP packages:

  1 lexical     type/token ratio, moving-average TTR, hapax ratio, mean word / sentence length
  2 coherence   adjacent-sentence word overlap (Jaccard), topic drift first vs. last third
  3 structure   sentence-length variance, punctuation variety, clause markers per sentence
  4 repetition  distinct-n, repeated n-gram fraction, longest repeated span, loop detection
  5 commitment  share of samples that end in a sentence terminator, numerals / proper-noun-like tokens

    python tools/analysis/analyze_text_quality.py --input analysis/my-run/generations.json
"""
from __future__ import annotations

import argparse
import json
import math
import re
from collections import Counter
from pathlib import Path
from statistics import mean, pvariance

from _common import write_json

WORD = re.compile(r"[A-Za-z0-9']+")
SENT = re.compile(r"(?<=[.!?])\s+")
CLAUSE = {"because", "although", "while", "which", "that", "when", "if", "since", "but", "however", "whereas", "unless"}


def words(t: str) -> list[str]:
    return [w.lower() for w in WORD.findall(t)]


def sentences(t: str) -> list[str]:
    return [s for s in SENT.split(t.strip()) if s]


def mattr(ws: list[str], window: int = 50) -> float:
    if len(ws) <= window:
        return len(set(ws)) / max(len(ws), 1)
    return mean(len(set(ws[i:i + window])) / window for i in range(len(ws) - window + 1))


def ngrams(ws: list[str], n: int) -> list[tuple]:
    return [tuple(ws[i:i + n]) for i in range(len(ws) - n + 1)]


def longest_repeat(ws: list[str]) -> int:
    """Length (in words) of the longest span that occurs at least twice."""
    best, n = 0, len(ws)
    for k in (32, 16, 8, 4, 2, 1):
        seen = set()
        for g in ngrams(ws, max(best, 0) + k):
            if g in seen:
                best += k
                break
            seen.add(g)
    return min(best, n)


def loop_period(ws: list[str], min_reps: int = 3) -> int:
    """Smallest period p such that the text ends in >= min_reps copies of a p-word unit (0 = none)."""
    for p in range(1, min(64, len(ws) // min_reps) + 1):
        unit = ws[-p:]
        if all(ws[-(r + 1) * p:len(ws) - r * p] == unit for r in range(min_reps)):
            return p
    return 0


def analyse(text: str) -> dict:
    ws, ss = words(text), sentences(text)
    if not ws:
        return {"empty": True}
    c = Counter(ws)
    lex = {"tokens": len(ws), "ttr": len(c) / len(ws), "mattr50": mattr(ws), "hapax_ratio": sum(v == 1 for v in c.values()) / len(c),
           "mean_word_len": mean(map(len, ws)), "mean_sentence_len": len(ws) / max(len(ss), 1)}
    sw = [set(words(s)) for s in ss if words(s)]
    adj = [len(a & b) / max(len(a | b), 1) for a, b in zip(sw, sw[1:])]
    third = max(len(ws) // 3, 1)
    first, last = Counter(ws[:third]), Counter(ws[-third:])
    dot = sum(first[k] * last[k] for k in first)
    drift = 1.0 - dot / (math.sqrt(sum(v * v for v in first.values())) * math.sqrt(sum(v * v for v in last.values())) + 1e-9)
    coh = {"adjacent_jaccard": mean(adj) if adj else 0.0, "topic_drift": drift}
    slen = [len(words(s)) for s in ss] or [0]
    struct = {"sentence_len_var": pvariance(slen) if len(slen) > 1 else 0.0,
              "punctuation_kinds": len(set(ch for ch in text if ch in ",;:—-()\"'!?.")),
              "clause_markers_per_sentence": sum(w in CLAUSE for w in ws) / max(len(ss), 1)}
    rep = {}
    for n in (1, 2, 3, 4):
        g = ngrams(ws, n)
        rep[f"distinct_{n}"] = len(set(g)) / max(len(g), 1)
    g4 = Counter(ngrams(ws, 4))
    rep["repeated_4gram_fraction"] = sum(v for v in g4.values() if v > 1) / max(sum(g4.values()), 1)
    rep["longest_repeated_span"] = longest_repeat(ws)
    rep["loop_period"] = loop_period(ws)
    commit = {"ends_terminated": text.rstrip()[-1:] in ".!?\"'", "numerals": sum(w.isdigit() for w in ws) / len(ws),
              "capitalised_mid_sentence": len(re.findall(r"(?<![.!?]\s)(?<!^)\b[A-Z][a-z]+", text)) / len(ws)}
    return {"lexical": lex, "coherence": coh, "structure": struct, "repetition": rep, "commitment": commit}


def aggregate(rows: list[dict]) -> dict:
    rows = [r for r in rows if not r.get("empty")]
    out: dict = {"n": len(rows)}
    if not rows:
        return out
    for layer in ("lexical", "coherence", "structure", "repetition", "commitment"):
        out[layer] = {k: mean(float(r[layer][k]) for r in rows) for k in rows[0][layer]}
    out["loop_rate"] = mean(1.0 if r["repetition"]["loop_period"] > 0 else 0.0 for r in rows)
    return out


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--input", required=True, help="generations.json of eval_generate / eval_via_server")
    ap.add_argument("--output", default=None)
    a = ap.parse_args()
    data = json.loads(Path(a.input).read_text())
    per_prompt, everything = [], []
    for g in data["generations"]:
        rows = [analyse(s) for s in g["samples"]]
        everything += rows
        per_prompt.append({"prompt": g["prompt"], "metrics": aggregate(rows)})
    out = {"run": data.get("run"), "overall": aggregate(everything), "per_prompt": per_prompt}
    dst = Path(a.output) if a.output else Path(a.input).with_name("text_quality.json")
    write_json(dst, out)
    print(f"{out['overall'].get('n', 0)} samples -> {dst}")


if __name__ == "__main__":
    main()
