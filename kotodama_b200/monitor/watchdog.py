"""Host watchdog for the training loop: names the rank and the phase that stalled.

The reference has no stall detection at all (``src/training/train.py`` only reacts to SIGTERM).
Here the loop announces each phase of a step (``data``, ``train_step``, ``loss_readback``,
``health_allreduce``, ``checkpoint`` ...); a daemon thread wakes a few times per limit and, when
the current phase has lasted longer than the limit, logs one error line with rank, step, phase
and elapsed time and calls the optional callback (a launcher can use it to mark the rank in a
store so that its peers stop before their next collective).  It never touches the GPU, so a hung
device cannot block it; with ``limit_s <= 0`` nothing is started.
"""
from __future__ import annotations

import logging
import threading
import time
from typing import Callable, Optional

logger = logging.getLogger(__name__)


class StepWatchdog:
    def __init__(self, limit_s: float, rank: int = 0, on_stall: Optional[Callable[[int, int, str, float], None]] = None,
                 poll_s: Optional[float] = None) -> None:
        self.limit_s = float(limit_s)
        self.rank = rank
        self.on_stall = on_stall
        self.stalls: list[tuple[int, str, float]] = []        # (step, phase, seconds) of every report
        self._lock = threading.Lock()
        self._step, self._phase, self._since = -1, "start", time.monotonic()
        self._reported = False
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        if self.limit_s > 0:
            self._poll = poll_s if poll_s is not None else max(0.01, min(1.0, self.limit_s / 4))
            self._thread = threading.Thread(target=self._run, name="kotodama-watchdog", daemon=True)
            self._thread.start()

    def phase(self, step: int, name: str) -> None:
        """The loop enters phase ``name`` of step ``step`` (also the heartbeat)."""
        with self._lock:
            self._step, self._phase, self._since = step, name, time.monotonic()
            self._reported = False

    def _run(self) -> None:
        while not self._stop.wait(self._poll):
            with self._lock:
                step, phase, dt = self._step, self._phase, time.monotonic() - self._since
                fire = dt > self.limit_s and not self._reported
                if fire:
                    self._reported = True
            if fire:
                self.stalls.append((step, phase, dt))
                logger.error("watchdog: rank %d has been in phase '%s' of step %d for %.1f s (limit %.1f s)",
                             self.rank, phase, step, dt, self.limit_s)
                if self.on_stall is not None:
                    try:
                        self.on_stall(self.rank, step, phase, dt)
                    except Exception:                          # noqa: BLE001 - a reporting hook must never raise
                        logger.exception("watchdog callback failed")

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
            self._thread = None
