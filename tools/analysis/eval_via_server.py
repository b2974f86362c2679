#!/usr/bin/env python
"""Track-3 generations through a running inference server (``serve.py``) instead of a local model.

    python tools/analysis/eval_via_server.py --url http://127.0.0.1:2222 --name owt-ddv1
    python tools/analysis/eval_via_server.py --url http://node2:2222 --name r --prompt-set extended --n-samples 3

Same output file as ``eval_generate.py``.  Counterpart of the reference's
``scripts/analysis/eval_via_server.py``.
"""
from __future__ import annotations

import argparse
import json
import time
import urllib.request

from _common import ROOT, load_yaml, run_dir, write_json


def post(url: str, body: dict, timeout: float = 600.0) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--url", required=True)
    ap.add_argument("--name", required=True)
    ap.add_argument("--prompt-set", default="standard")
    ap.add_argument("--prompts-file", default=str(ROOT / "configs" / "prompts.yaml"))
    ap.add_argument("--n-samples", type=int, default=1)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--max-tokens", type=int, default=256)
    ap.add_argument("--output-dir", default="analysis")
    a = ap.parse_args()
    base = a.url.rstrip("/")
    with urllib.request.urlopen(base + "/info", timeout=30) as r:
        info = json.loads(r.read())
    prompts = load_yaml(a.prompts_file)[a.prompt_set]
    t0 = time.time()
    gens = []
    for p in prompts:
        samples = []
        for _ in range(a.n_samples):
            res = post(base + "/generate", {"prompt": p, "max_tokens": a.max_tokens, "temperature": a.temperature,
                                            "top_k": a.top_k, "top_p": a.top_p})
            samples.append(res.get("text", ""))
        gens.append({"prompt": p, "samples": samples})
    out = {"run": a.name, "server": base, "server_info": info,
           "config": {"temperature": a.temperature, "top_k": a.top_k, "top_p": a.top_p, "max_tokens": a.max_tokens,
                      "n_samples": a.n_samples, "prompt_set": a.prompt_set},
           "generations": gens, "generation_s": round(time.time() - t0, 2)}
    write_json(run_dir(a.output_dir, a.name) / "generations.json", out)
    print(f"{a.name}: {len(gens)} prompts -> {run_dir(a.output_dir, a.name) / 'generations.json'}")


if __name__ == "__main__":
    main()
