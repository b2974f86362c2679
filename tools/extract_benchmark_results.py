#!/usr/bin/env python
"""Summarise a training log: tok/s percentiles (warm-up lines skipped), device-timed tok/s when
present, peak memory and the last loss.  Reads the canonical step line
``step=... | loss=... | ... | tok/s=... | ... | gpu_mem=...GB``."""
import json
import re
import statistics
import sys


def summarise(path: str, skip: int = 3) -> dict:
    toks, dev, mem, loss = [], [], [], []
    for line in open(path, errors="replace"):
        m = re.search(r"tok/s=(\d+)", line)
        if m and "step=" in line:
            toks.append(float(m.group(1)))
            g = re.search(r"gpu_mem=([\d.]+)GB", line)
            if g:
                mem.append(float(g.group(1)))
            l = re.search(r"loss=([\d.]+)", line)
            if l:
                loss.append(float(l.group(1)))
        d = re.search(r"device-timed: [\d.]+ ms/step, (\d+) tok/s", line)
        if d:
            dev.append(float(d.group(1)))
    steady = toks[skip:] or toks
    out = {"log": path, "lines": len(toks)}
    if steady:
        s = sorted(steady)
        out.update(tok_s_p5=s[int(0.05 * (len(s) - 1))], tok_s_median=statistics.median(s),
                   tok_s_p95=s[int(0.95 * (len(s) - 1))])
    if dev[skip:] or dev:
        out["device_tok_s_median"] = statistics.median(dev[skip:] or dev)
    if mem:
        out["gpu_mem_gb_max"] = max(mem)
    if loss:
        out["loss_last"] = loss[-1]
    return out


if __name__ == "__main__":
    for p in sys.argv[1:]:
        print(json.dumps(summarise(p)))
