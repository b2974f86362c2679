#!/usr/bin/env python
"""Summarise a chrome trace written by ``--profile`` (or ``tools/profile_step.py --trace``):

* device kernels (events with ``cat == "kernel"``): total time per kernel name, calls, mean, share of the traced
  device time, and how much of it the listed rows cover;
* host side (``cpu_op`` and ``user_annotation`` events): total time and calls per op, which shows where the launching
  thread spends its time (``--cpu N`` rows, 15 by default).

    python tools/parse_profile.py trace.json [top kernels] [--cpu N]

Same figures as the reference's ``tools/parse_profile.py``.
"""
import json
import sys
from collections import defaultdict


def _aggregate(path: str, cats: tuple[str, ...]) -> list[tuple[str, float, int]]:
    with open(path) as fh:
        raw = json.load(fh)
    events = raw.get("traceEvents", raw) if isinstance(raw, dict) else raw
    tot, cnt = defaultdict(float), defaultdict(int)
    for e in events:
        if e.get("cat") in cats and e.get("dur"):
            tot[e.get("name", "unknown")] += e["dur"]
            cnt[e.get("name", "unknown")] += 1
    return sorted(((n, t, cnt[n]) for n, t in tot.items()), key=lambda r: -r[1])


def parse(path: str, top: int = 40) -> list[tuple[str, float, int]]:
    """(kernel name, total microseconds, calls), longest first."""
    return _aggregate(path, ("kernel",))[:top]


def parse_cpu(path: str, top: int = 15) -> list[tuple[str, float, int]]:
    """(op name, total microseconds, calls) of the host-side ops and annotations, longest first."""
    return _aggregate(path, ("cpu_op", "user_annotation"))[:top]


if __name__ == "__main__":
    argv = sys.argv[1:]
    cpu_rows = 15
    if "--cpu" in argv:
        i = argv.index("--cpu")
        cpu_rows = int(argv[i + 1])
        del argv[i:i + 2]
    every = _aggregate(argv[0], ("kernel",))
    rows = every[: int(argv[1]) if len(argv) > 1 else 40]
    total = sum(r[1] for r in every) or 1.0
    print(f"{'kernel':<90}{'ms':>10}{'calls':>8}{'mean us':>10}{'share':>8}")
    for n, t, c in rows:
        print(f"{n[:88]:<90}{t / 1e3:>10.2f}{c:>8}{t / max(c, 1):>10.1f}{100 * t / total:>7.1f}%")
    print(f"device time {total / 1e3:.2f} ms over {len(every)} kernels; the rows above cover {100 * sum(r[1] for r in rows) / total:.1f}%")
    host = parse_cpu(argv[0], cpu_rows)
    if host:
        print(f"\n{'host op':<90}{'ms':>10}{'calls':>8}")
        for n, t, c in host:
            print(f"{n[:88]:<90}{t / 1e3:>10.2f}{c:>8}")
