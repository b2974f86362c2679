#!/usr/bin/env python
"""Track-3 generations through a running inference server (``serve.py``) instead of a local model.

    python tools/analysis/eval_via_server.py --url http://127.0.0.1:2222 --name owt-ddv1
    python tools/analysis/eval_via_server.py --url http://node2:2222 --name r --prompt-set extended --n-samples 3 \\
        --concurrency 16 --temperature 0.8 --top-p 0.9

The server batches whatever is in flight (continuous batching), so the requests of a prompt set are
sent ``--concurrency`` at a time from a thread pool; every request is retried on connection errors and
5xx answers (``--retries``), and the tool first waits until ``/health`` answers (``--wait``).  Besides
the samples the output records the server's ``/info``, per-request latency and tokens per second, and
the aggregate throughput of the evaluation.

Same output file as ``eval_generate.py`` (``<output-dir>/<name>/generations.json``), so
``analyze_text_quality.py`` and ``generate_report.py`` read either.  Counterpart of the reference's
``scripts/analysis/eval_via_server.py``.
"""
from __future__ import annotations

import argparse
import json
import statistics
import time
import urllib.error
import urllib.request
from concurrent.futures import ThreadPoolExecutor
from pathlib import Path
from typing import Any

from _common import ROOT, load_yaml, run_dir, write_json


def get_json(url: str, timeout: float = 30.0) -> dict:
    with urllib.request.urlopen(url, timeout=timeout) as r:
        return json.loads(r.read())


def post_json(url: str, body: dict, timeout: float = 600.0) -> dict:
    req = urllib.request.Request(url, data=json.dumps(body).encode(), headers={"Content-Type": "application/json"})
    with urllib.request.urlopen(req, timeout=timeout) as r:
        return json.loads(r.read())


def wait_for_server(base: str, seconds: float) -> None:
    """Poll /health until the server answers or the time is up."""
    deadline = time.time() + seconds
    last: Exception | None = None
    while True:
        try:
            if get_json(base + "/health", timeout=5).get("status") == "ok":
                return
        except (urllib.error.URLError, OSError, ValueError) as e:
            last = e
        if time.time() >= deadline:
            raise SystemExit(f"{base}/health did not answer within {seconds:.0f}s ({last})")
        time.sleep(1.0)


def generate_one(base: str, body: dict, retries: int, timeout: float) -> dict[str, Any]:
    """One /generate call; retried on connection errors and 5xx, not on 4xx (a bad request stays bad)."""
    err, made = "", 0
    for attempt in range(retries + 1):
        made = attempt + 1
        t0 = time.time()
        try:
            res = post_json(base + "/generate", body, timeout)
            return {"text": res.get("text", ""), "prompt_tokens": res.get("prompt_tokens"),
                    "completion_tokens": res.get("completion_tokens"), "latency_s": round(time.time() - t0, 3),
                    "tokens_per_second": res.get("tokens_per_second"), "attempts": attempt + 1}
        except urllib.error.HTTPError as e:
            err = f"HTTP {e.code}: {e.read()[:200].decode(errors='replace')}"
            if e.code < 500:
                break
        except (urllib.error.URLError, OSError, ValueError) as e:
            err = str(e)
        time.sleep(min(2.0 ** attempt, 10.0))
    return {"text": "", "error": err, "latency_s": None, "attempts": made}


def main() -> None:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--url", required=True, help="server address, e.g. http://node2:2222")
    ap.add_argument("--name", required=True, help="run name of the output")
    ap.add_argument("--prompt-set", default="extended")
    ap.add_argument("--prompts-file", default=str(ROOT / "configs" / "prompts.yaml"))
    ap.add_argument("--n-samples", type=int, default=3)
    ap.add_argument("--temperature", type=float, default=0.7)
    ap.add_argument("--top-k", type=int, default=50)
    ap.add_argument("--top-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--max-tokens", type=int, default=512)
    ap.add_argument("--concurrency", type=int, default=8, help="requests in flight")
    ap.add_argument("--retries", type=int, default=2)
    ap.add_argument("--timeout", type=float, default=600.0, help="seconds per request")
    ap.add_argument("--wait", type=float, default=0.0, help="seconds to wait for /health before starting")
    ap.add_argument("--output-dir", default="analysis")
    ap.add_argument("--output", "-o", default=None, help="output file (default: <output-dir>/<name>/generations.json)")
    a = ap.parse_args()
    base = a.url.rstrip("/")
    if a.wait > 0:
        wait_for_server(base, a.wait)
    info = get_json(base + "/info")
    sets = load_yaml(a.prompts_file)
    if a.prompt_set not in sets or not isinstance(sets[a.prompt_set], list):
        raise SystemExit(f"unknown prompt set '{a.prompt_set}'; {a.prompts_file} has {sorted(sets)}")
    prompts = sets[a.prompt_set]
    body = {"max_new_tokens": a.max_tokens, "temperature": a.temperature, "top_k": a.top_k, "top_p": a.top_p,
            "repetition_penalty": a.repetition_penalty}
    jobs = [(pi, si) for pi in range(len(prompts)) for si in range(a.n_samples)]
    t0 = time.time()
    with ThreadPoolExecutor(max_workers=max(1, a.concurrency)) as pool:
        results = list(pool.map(lambda j: generate_one(base, {"prompt": prompts[j[0]], **body}, a.retries, a.timeout), jobs))
    wall = time.time() - t0
    gens = []
    for pi, p in enumerate(prompts):
        mine = [r for (qi, _), r in zip(jobs, results) if qi == pi]
        gens.append({"prompt": p, "samples": [r["text"] for r in mine],
                     "requests": [{k: v for k, v in r.items() if k != "text"} for r in mine]})
    ok = [r for r in results if "error" not in r]
    lat = [r["latency_s"] for r in ok if r["latency_s"] is not None]
    toks = sum(r.get("completion_tokens") or 0 for r in ok)
    stats = {"requests": len(results), "failed": len(results) - len(ok), "wall_s": round(wall, 2), "completion_tokens": toks,
             "aggregate_tokens_per_second": round(toks / wall, 1) if wall > 0 else None,
             "latency_s_median": round(statistics.median(lat), 3) if lat else None,
             "latency_s_max": round(max(lat), 3) if lat else None, "concurrency": a.concurrency}
    out = {"run": a.name, "server": base, "server_info": info,
           "config": {"temperature": a.temperature, "top_k": a.top_k, "top_p": a.top_p, "max_tokens": a.max_tokens,
                      "repetition_penalty": a.repetition_penalty, "n_samples": a.n_samples, "prompt_set": a.prompt_set},
           "generations": gens, "generation_s": round(wall, 2), "server_stats": stats}
    path = Path(a.output) if a.output else run_dir(a.output_dir, a.name) / "generations.json"
    write_json(path, out)
    print(f"{a.name}: {len(prompts)} prompts x {a.n_samples} samples in {wall:.1f}s "
          f"({stats['aggregate_tokens_per_second']} tok/s aggregate, {stats['failed']} failed) -> {path}")
    if stats["failed"]:
        first = next(r for r in results if "error" in r)
        print(f"  first error: {first['error']}")


if __name__ == "__main__":
    main()
