#!/usr/bin/env python
"""Concept-geometry extraction (track 6a): residual-stream activations of concept words (months,
weekdays, digits, compass points, states, antonym pairs, ...; ``configs/concepts.yaml``) under
several sentence templates, at every layer.

For every (template, item) the sentence is tokenised, the item's token span inside it is located,
one forward pass is run, and three views of the residual stream are kept per layer:

  acts      the state at the item's LAST token (what a causal model has once it has read the word)
  pooled    the mean state over the item's tokens (multi-token items)
  last_tok  the state at the last token of the sentence (what the model carries forward)

    python tools/analysis/extract_concept_geometry.py --checkpoint ckpt.pt --name run
    python tools/analysis/extract_concept_geometry.py --checkpoints a,b --concept-sets months,digits --tier 1
    python tools/analysis/extract_concept_geometry.py --checkpoint ckpt.pt --validate-only       # tokenisation report

Writes ``<output-dir>/<run>/concept_geometry/<set>.npz`` (``acts``, ``pooled``, ``last_tok``:
``[templates, items, layers+1, D]`` float32; ``token_counts`` ``[templates, items]``) and ``meta.json``
(kind, tier, items, coordinates, the tokenisation report).  Counterpart of the reference's
``scripts/analysis/extract_concept_geometry.py``.
"""
from __future__ import annotations

import argparse
import time
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np
import torch
from _common import ROOT, add_checkpoint_args, load_yaml, open_model, run_dir, select_checkpoints, tokenizer, write_json

from kotodama_b200.eval import forward_with_states


@dataclass
class ConceptSet:
    name: str
    kind: str
    items: list[str]
    tier: int = 1
    category: str = "word"
    coordinates: Optional[dict[str, list[float]]] = None
    extra: dict[str, Any] = field(default_factory=dict)


def load_concepts(path: str) -> tuple[list[str], dict[str, ConceptSet]]:
    spec = load_yaml(path)
    sets = {}
    for name, s in spec["sets"].items():
        known = {"kind", "items", "tier", "category", "coordinates"}
        sets[name] = ConceptSet(name, s["kind"], [str(i) for i in s["items"]], int(s.get("tier", 1)), str(s.get("category", "word")),
                                s.get("coordinates"), {k: v for k, v in s.items() if k not in known})
        if sets[name].kind == "paired" and len(sets[name].items) % 2:
            raise SystemExit(f"concept set '{name}' is 'paired' but has an odd number of items")
        if sets[name].kind == "geographic":
            missing = [i for i in sets[name].items if i not in (sets[name].coordinates or {})]
            if missing:
                raise SystemExit(f"concept set '{name}' is 'geographic' but has no coordinates for {missing}")
    return list(spec["templates"]), sets


def fill(template: str, item: str, category: str) -> tuple[str, int]:
    """The sentence and the character offset of the item in it."""
    marked = template.replace("{category}", category)
    at = marked.index("{}")
    return marked.replace("{}", item, 1), at


def _common_prefix(a: list[int], b: list[int]) -> int:
    n = 0
    while n < len(a) and n < len(b) and a[n] == b[n]:
        n += 1
    return n


def locate(tok: Any, template: str, item: str, category: str) -> tuple[list[int], int, int]:
    """Token ids of the sentence and the inclusive token span [start, end] of the item.

    The span is found from encodings of growing prefixes: tokens the encoding of "text before the item"
    shares with the full encoding are before the span; the encoding of "text up to the item's end" gives
    the span's last token.  Tokenisers that merge across the boundary (a leading space glued to the word,
    byte-pair merges) shorten the shared part, so the span then starts at the first token that differs -
    which is the token holding the item's first character."""
    text, at = fill(template, item, category)
    full = tok.encode(text)
    if not full:
        raise ValueError(f"empty encoding for '{text}'")
    upto = tok.encode(text[: at + len(item)])
    before = tok.encode(text[:at]) if at > 0 else []
    end = min(max(_common_prefix(full, upto) - 1, 0), len(full) - 1)
    if at + len(item) == len(text):
        end = len(full) - 1
    start = min(_common_prefix(full, before), end) if at > 0 else 0
    # a special first token (BOS) belongs to no word
    if at == 0 and len(full) > 1 and end > 0 and tok.encode("") == full[:1]:
        start = 1
    return full, start, end


def tokenisation_report(tok: Any, templates: list[str], sets: dict[str, ConceptSet]) -> dict[str, Any]:
    """Which items take more than one token, per set (multi-token items make `acts` and `pooled` differ)."""
    rep = {}
    for name, cs in sets.items():
        multi = {}
        for it in cs.items:
            counts = []
            for t in templates:
                _, s, e = locate(tok, t, it, cs.category)
                counts.append(e - s + 1)
            if max(counts) > 1:
                multi[it] = counts
        rep[name] = {"items": len(cs.items), "multi_token_items": len(multi), "token_counts": multi}
    return rep


@torch.no_grad()
def extract_set(model: Any, tok: Any, cs: ConceptSet, templates: list[str], device: str) -> dict[str, np.ndarray]:
    T, n = len(templates), len(cs.items)
    L, D = model.config.num_layers, model.config.hidden_size
    acts = np.zeros((T, n, L + 1, D), dtype=np.float32)
    pooled, last = np.zeros_like(acts), np.zeros_like(acts)
    counts = np.zeros((T, n), dtype=np.int32)
    limit = model.config.max_position_embeddings
    for ti, t in enumerate(templates):
        for ii, it in enumerate(cs.items):
            ids, s, e = locate(tok, t, it, cs.category)
            ids, s, e = ids[:limit], min(s, limit - 1), min(e, limit - 1)
            res = forward_with_states(model, torch.tensor([ids], device=device))
            for l, st in enumerate(res.states):
                x = st[0].float()
                acts[ti, ii, l] = x[e].cpu().numpy()
                pooled[ti, ii, l] = x[s:e + 1].mean(0).cpu().numpy()
                last[ti, ii, l] = x[-1].cpu().numpy()
            counts[ti, ii] = e - s + 1
    return {"acts": acts, "pooled": pooled, "last_tok": last, "token_counts": counts}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_checkpoint_args(ap)
    ap.add_argument("--concepts-file", "--concepts-config", dest="concepts_file", default=str(ROOT / "configs" / "concepts.yaml"))
    ap.add_argument("--concept-sets", default=None, help="comma-separated names (default: all)")
    ap.add_argument("--tier", type=int, default=None, help="only sets of this tier or lower")
    ap.add_argument("--templates", default=None, help="comma-separated template indices (default: all)")
    ap.add_argument("--validate-only", action="store_true", help="print the tokenisation report and exit (no model is loaded)")
    a = ap.parse_args()
    templates, sets = load_concepts(a.concepts_file)
    if a.templates:
        templates = [templates[int(i)] for i in a.templates.split(",")]
    chosen = [s.strip() for s in a.concept_sets.split(",")] if a.concept_sets else list(sets)
    unknown = [s for s in chosen if s not in sets]
    if unknown:
        raise SystemExit(f"unknown concept sets {unknown}; the file has {sorted(sets)}")
    if a.tier is not None:
        chosen = [s for s in chosen if sets[s].tier <= a.tier]
    sets = {s: sets[s] for s in chosen}
    tok = tokenizer(a.tokenizer)
    report = tokenisation_report(tok, templates, sets)
    for name, r in report.items():
        print(f"  {name}: {r['multi_token_items']}/{r['items']} items take more than one token in some template")
    if a.validate_only:
        return
    for run, kw in select_checkpoints(a):
        t0 = time.time()
        model, _ = open_model(kw, a.device)
        d = run_dir(a.output_dir, run, "concept_geometry")
        meta: dict[str, Any] = {"run": run, "templates": templates, "layers": model.config.num_layers,
                                "hidden_size": model.config.hidden_size, "tokenisation": report, "sets": {}}
        for name, cs in sets.items():
            arrays = extract_set(model, tok, cs, templates, a.device)
            np.savez_compressed(d / f"{name}.npz", **arrays)
            meta["sets"][name] = {"kind": cs.kind, "tier": cs.tier, "category": cs.category, "items": cs.items,
                                  **({"coordinates": [cs.coordinates[i] for i in cs.items]} if cs.coordinates else {}), **cs.extra}
        write_json(d / "meta.json", meta)
        print(f"{run}: {len(sets)} concept sets x {len(templates)} templates -> {d} ({time.time() - t0:.1f}s)")
        del model


if __name__ == "__main__":
    main()
