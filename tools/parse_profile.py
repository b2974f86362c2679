#!/usr/bin/env python
"""Aggregate kernel time from a chrome trace written by ``--profile`` (events with ``cat == "kernel"``):
total per kernel name, share of the traced device time, call counts."""
import json
import sys
from collections import defaultdict


def parse(path: str, top: int = 40) -> list[tuple[str, float, int]]:
    raw = json.load(open(path))
    events = raw["traceEvents"] if isinstance(raw, dict) else raw
    tot, cnt = defaultdict(float), defaultdict(int)
    for e in events:
        if e.get("cat") == "kernel" and "dur" in e:
            tot[e["name"]] += e["dur"]
            cnt[e["name"]] += 1
    rows = sorted(((n, t, cnt[n]) for n, t in tot.items()), key=lambda r: -r[1])
    return rows[:top]


if __name__ == "__main__":
    rows = parse(sys.argv[1], int(sys.argv[2]) if len(sys.argv) > 2 else 40)
    total = sum(r[1] for r in rows) or 1.0
    print(f"{'kernel':<90}{'ms':>10}{'calls':>8}{'share':>8}")
    for n, t, c in rows:
        print(f"{n[:88]:<90}{t / 1e3:>10.2f}{c:>8}{100 * t / total:>7.1f}%")
