"""Profiling window for the training loop and NVTX / CUDA-event phase timing.

``--profile`` (``src/training/train.py:540-551,569-580,750-774`` in the reference): on rank 0 a
``torch.profiler`` session starts at ``--profile_start_step``, steps once per iteration and after
``--profile_steps`` writes ``chrome_trace.json`` and ``profile_summary.txt`` (top kernels by device
time, then by FLOPs) under ``--profile_dir`` (default ``<checkpoint_dir>/profile``).
:class:`PhaseTimer` brackets named phases with CUDA events (device time, no host sync until
read) and NVTX ranges so the same names show up in Nsight captures.
"""
from __future__ import annotations

import contextlib
import logging
from collections import defaultdict
from pathlib import Path
from typing import Any, Iterator

import torch

logger = logging.getLogger(__name__)


class StepProfiler:
    def __init__(self, args: Any, enabled: bool) -> None:
        self.enabled = bool(enabled)
        self.start = getattr(args, "profile_start_step", 50)
        self.end = self.start + getattr(args, "profile_steps", 20)
        self.dir = Path(getattr(args, "profile_dir", None) or getattr(args, "checkpoint_dir", ".")) / "profile"
        self._prof = None
        if self.enabled:
            self.dir.mkdir(parents=True, exist_ok=True)
            logger.info("Profiler enabled: steps %d-%d, output: %s", self.start, self.end, self.dir)

    def step_begin(self, step: int) -> None:
        if not self.enabled or self._prof is not None or step != self.start:
            return
        acts = [torch.profiler.ProfilerActivity.CPU]
        if torch.cuda.is_available():
            acts.append(torch.profiler.ProfilerActivity.CUDA)
        self._prof = torch.profiler.profile(activities=acts, record_shapes=True, with_flops=True, profile_memory=True)
        self._prof.__enter__()
        logger.info("Profiler started at step %d", step)

    def step_end(self, step: int) -> None:
        if self._prof is None:
            return
        self._prof.step()
        if step < self.end:
            return
        self._prof.__exit__(None, None, None)
        trace, summary = self.dir / "chrome_trace.json", self.dir / "profile_summary.txt"
        try:
            self._prof.export_chrome_trace(str(trace))
            sort = "cuda_time_total" if torch.cuda.is_available() else "cpu_time_total"
            with open(summary, "w") as fh:
                fh.write(self._prof.key_averages().table(sort_by=sort, row_limit=60))
                fh.write("\n\n--- FLOPS ---\n\n")
                fh.write(self._prof.key_averages().table(sort_by="flops", row_limit=20))
            logger.info("Profiler stopped at step %d. Trace: %s, Summary: %s", step, trace, summary)
        except Exception as e:          # noqa: BLE001 - profiling must not end the run
            logger.warning("Profiler export failed: %s", e)
        self._prof = None


class PhaseTimer:
    """``with timer.phase("forward"): ...`` — device-timed phases (falls back to host time on CPU)."""

    def __init__(self, cuda: bool) -> None:
        self.cuda = cuda and torch.cuda.is_available()
        self._events: list[tuple[str, Any, Any]] = []
        self._host: dict[str, float] = defaultdict(float)

    @contextlib.contextmanager
    def phase(self, name: str) -> Iterator[None]:
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            torch.cuda.nvtx.range_push(name)
            e0.record()
            try:
                yield
            finally:
                e1.record()
                torch.cuda.nvtx.range_pop()
                self._events.append((name, e0, e1))
        else:
            import time
            t0 = time.perf_counter()
            try:
                yield
            finally:
                self._host[name] += (time.perf_counter() - t0) * 1e3

    def totals_ms(self) -> dict[str, float]:
        out = dict(self._host)
        if self.cuda:
            torch.cuda.synchronize()
            for name, e0, e1 in self._events:
                out[name] = out.get(name, 0.0) + e0.elapsed_time(e1)
            self._events.clear()
        return out
