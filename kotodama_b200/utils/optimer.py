"""Per-op timing: wraps an ops backend so that every call is bracketed by CUDA events (host clock
where there is no GPU: the CPU back end runs its ops synchronously) and aggregated by op name.  Used by
``bench.py --op-times``, ``tools/profile_step.py`` and the kernel benchmarks; adds two event records per
call, so totals are slightly above an untimed run."""
from __future__ import annotations

import time
from collections import defaultdict
from typing import Any

import torch


class TimedOps:
    def __init__(self, inner: Any, prefix: str = "") -> None:
        self._inner = inner
        self._prefix = prefix
        self._events: list[tuple[str, Any, Any]] = []      # (label, start, end): CUDA events, or host seconds
        self.enabled = True
        self._cuda = torch.cuda.is_available()

    def __getattr__(self, name: str) -> Any:
        attr = getattr(self._inner, name)
        if not callable(attr) or name.startswith("_") or name in ("check_status", "status", "allocator", "attach"):
            return attr

        def wrapped(*a: Any, **k: Any) -> Any:
            if not self.enabled:
                return attr(*a, **k)
            if self._cuda:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
                out = attr(*a, **k)
                e1.record()
            else:
                e0 = time.perf_counter()
                out = attr(*a, **k)
                e1 = time.perf_counter()
            label = self._prefix + name
            if name.startswith("gemm") and a:
                label = f"{name}[{'x'.join(map(str, a[0].shape))}|{'x'.join(map(str, a[1].shape))}]"
            self._events.append((label, e0, e1))
            return out

        return wrapped

    def reset(self) -> None:
        self._events.clear()

    def summary(self) -> list[tuple[str, float, int]]:
        if self._cuda:
            torch.cuda.synchronize()
        tot: dict[str, float] = defaultdict(float)
        cnt: dict[str, int] = defaultdict(int)
        for name, e0, e1 in self._events:
            tot[name] += e0.elapsed_time(e1) if self._cuda else (e1 - e0) * 1e3
            cnt[name] += 1
        return sorted(((n, t, cnt[n]) for n, t in tot.items()), key=lambda x: -x[1])

    def table(self, steps: int = 1) -> str:
        rows = self.summary()
        total = sum(t for _, t, _ in rows)
        lines = [f"{'op':<64}{'ms/step':>10}{'calls/step':>12}{'share':>8}"]
        for n, t, c in rows:
            lines.append(f"{n:<64}{t / steps:>10.2f}{c / steps:>12.1f}{100 * t / max(total, 1e-9):>7.1f}%")
        lines.append(f"{'TOTAL (sum of op times; nested ops counted twice)':<64}{total / steps:>10.2f}")
        return "\n".join(lines)
