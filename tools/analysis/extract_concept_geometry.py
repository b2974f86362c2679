#!/usr/bin/env python
"""Concept-geometry extraction (track 6a): residual-stream activations at the last token of each
concept word (months, weekdays, digits, ...; ``configs/concepts.yaml``) under several templates,
at every layer.

    python tools/analysis/extract_concept_geometry.py --checkpoint ckpt.pt --name run
    python tools/analysis/extract_concept_geometry.py --checkpoints a,b --concept-sets months,digits --tier 1

Writes ``<output-dir>/<run>/concept_geometry/<set>.npz`` with ``acts [templates, items, layers+1, D]``
and a ``meta.json``.  Counterpart of the reference's ``scripts/analysis/extract_concept_geometry.py``.
"""
from __future__ import annotations

import argparse

import numpy as np
import torch
from _common import ROOT, add_checkpoint_args, load_yaml, open_model, run_dir, select_checkpoints, tokenizer, write_json

from kotodama_b200.eval import forward_with_states


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    add_checkpoint_args(ap)
    ap.add_argument("--concepts-file", default=str(ROOT / "configs" / "concepts.yaml"))
    ap.add_argument("--concept-sets", default=None)
    ap.add_argument("--tier", type=int, default=None)
    a = ap.parse_args()
    spec = load_yaml(a.concepts_file)
    templates, sets = spec["templates"], spec["sets"]
    chosen = [s.strip() for s in a.concept_sets.split(",")] if a.concept_sets else list(sets)
    if a.tier is not None:
        chosen = [s for s in chosen if sets[s].get("tier", 1) <= a.tier]
    tok = tokenizer(a.tokenizer)
    for run, kw in select_checkpoints(a):
        model, _ = open_model(kw, a.device)
        d = run_dir(a.output_dir, run, "concept_geometry")
        meta = {"run": run, "templates": templates, "sets": {}}
        for name in chosen:
            items = sets[name]["items"]
            acts = []
            for t in templates:
                row = []
                for it in items:
                    ids = torch.tensor([tok.encode(t.format(it))], device=a.device)
                    res = forward_with_states(model, ids)
                    row.append(torch.stack([s[0, -1].float().cpu() for s in res.states]).numpy())
                acts.append(np.stack(row))
            np.savez_compressed(d / f"{name}.npz", acts=np.stack(acts).astype(np.float32))
            meta["sets"][name] = {"kind": sets[name]["kind"], "items": items}
        write_json(d / "meta.json", meta)
        print(f"{run}: {chosen} -> {d}")


if __name__ == "__main__":
    main()
