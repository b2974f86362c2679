"""Metrics logging: namespaced metrics to wandb (when usable) and always to JSONL, the
canonical step line that the run tooling parses, and the optional job-scheduler hook.

Parity: ``src/monitoring/wandb_callback.py:34-258`` (keys ``train/*``, ``optim/*``, ``perf/*``,
``data/*``, ``geo/*``; ``metrics.jsonl`` and ``geo_metrics.jsonl``; loss / RankMe slopes over
sliding windows; one wandb commit per step) and the step line at
``src/training/train.py:674-689`` (tools read ``tok/s=``, ``gpu_mem=`` and ``loss=`` from it).
Logging never raises into the training loop.
"""
from __future__ import annotations

import json
import logging
import math
import os
import time
from collections import deque
from pathlib import Path
from typing import Any, Optional

logger = logging.getLogger(__name__)

STEP_LINE = ("step=%d/%d | loss=%.4f | z_loss=%.6f | grad_norm=%.3f | muon_lr=%.6f | adamw_lr=%.6f | "
             "tok/s=%.0f | it/s=%.2f | tokens=%.3fB | gpu_mem=%.1fGB")


def format_step_line(step: int, total: int, loss: float, z_loss: float, grad_norm: float, muon_lr: float,
                     adamw_lr: float, tok_s: float, it_s: float, tokens: int, gpu_mem_gb: float) -> str:
    return STEP_LINE % (step, total, loss, z_loss, grad_norm, muon_lr, adamw_lr, tok_s, it_s, tokens / 1e9, gpu_mem_gb)


def linear_slope(points: list[tuple[float, float]]) -> float:
    """Least-squares slope through ``(x, y)`` points; 0 for fewer than two or a degenerate x range."""
    n = len(points)
    if n < 2:
        return 0.0
    mx = sum(p[0] for p in points) / n
    my = sum(p[1] for p in points) / n
    den = sum((p[0] - mx) ** 2 for p in points)
    if den < 1e-10:
        return 0.0
    return sum((p[0] - mx) * (p[1] - my) for p in points) / den


class WandbLogger:
    def __init__(self, project: str = "luxia-base", run_name: Optional[str] = None,
                 config: Optional[dict[str, Any]] = None, log_dir: str = "logs", enabled: bool = True,
                 tags: Optional[list[str]] = None, use_wandb: bool = True) -> None:
        self.enabled = enabled
        self._run = None
        self._files: dict[str, Any] = {}
        self._loss_hist: deque = deque(maxlen=100)
        self._rankme_hist: deque = deque(maxlen=50)
        if not enabled:
            return
        d = Path(log_dir)
        d.mkdir(parents=True, exist_ok=True)
        self.metrics_path, self.geo_path = d / "metrics.jsonl", d / "geo_metrics.jsonl"
        self._files = {"metrics": open(self.metrics_path, "a"), "geo": open(self.geo_path, "a")}
        if use_wandb:
            try:
                import wandb
                if not os.environ.get("WANDB_API_KEY"):
                    os.environ.setdefault("WANDB_MODE", "offline")
                self._run = wandb.init(project=project, name=run_name, config=config or {},
                                       tags=tags or ["pretraining", "luxia-base"], resume="allow")
            except Exception as e:      # noqa: BLE001 - wandb is optional
                logger.warning("wandb unavailable (%s): logging to JSONL only", e)
                self._run = None

    def _write(self, which: str, record: dict[str, Any]) -> None:
        f = self._files.get(which)
        if f is None:
            return
        try:
            f.write(json.dumps(record) + "\n")
            f.flush()
        except Exception as e:          # noqa: BLE001
            logger.debug("JSONL write failed: %s", e)

    def _log(self, step: int, metrics: dict[str, Any]) -> None:
        if not self.enabled:
            return
        self._write("metrics", {"step": step, "timestamp": time.time(), **metrics})
        if self._run is not None:
            try:
                import wandb
                wandb.log(metrics, step=step, commit=False)
            except Exception as e:      # noqa: BLE001
                logger.debug("wandb log failed: %s", e)

    def log_step(self, step: int, loss: float, z_loss: float, grad_norm: float, muon_lr: float, adamw_lr: float,
                 tokens_per_sec: float, tokens_consumed: int, gpu_mem_gb: float, step_time_s: float,
                 iters_per_sec: float = 0.0) -> None:
        if not self.enabled:
            return
        self._loss_hist.append((step, loss))
        m = {"train/loss": loss, "train/z_loss": z_loss, "train/perplexity": math.exp(min(loss, 20.0)),
             "train/grad_norm": grad_norm, "optim/muon_lr": muon_lr, "optim/adamw_lr": adamw_lr,
             "perf/tokens_per_sec": tokens_per_sec, "perf/iters_per_sec": iters_per_sec,
             "perf/gpu_mem_gb": gpu_mem_gb, "perf/step_time_s": step_time_s,
             "data/tokens_consumed": tokens_consumed, "data/tokens_consumed_B": tokens_consumed / 1e9}
        if len(self._loss_hist) >= 10:
            m["train/loss_slope"] = linear_slope(list(self._loss_hist))
        self._log(step, m)

    def log_geo(self, step: int, geo_metrics: dict[str, float]) -> None:
        if not self.enabled or not geo_metrics:
            return
        r = geo_metrics.get("geo/rankme_last")
        if r is not None:
            self._rankme_hist.append((step, r))
            if len(self._rankme_hist) >= 5:
                geo_metrics["geo/rankme_slope"] = linear_slope(list(self._rankme_hist))
        self._write("geo", {"step": step, "timestamp": time.time(), **geo_metrics})
        self._log(step, geo_metrics)

    def log_custom(self, step: int, metrics: dict[str, Any]) -> None:
        self._log(step, metrics)

    def commit(self, step: int) -> None:
        if self._run is not None:
            try:
                import wandb
                wandb.log({}, step=step, commit=True)
            except Exception:           # noqa: BLE001
                pass

    def finish(self) -> None:
        if self._run is not None:
            try:
                import wandb
                wandb.finish()
            except Exception:           # noqa: BLE001
                pass
        for f in self._files.values():
            try:
                f.close()
            except Exception:           # noqa: BLE001
                pass
        self._files = {}


_scheduler_client = None


def scheduler_hook(step: int, **metrics: float) -> None:
    """Fire-and-forget POST of metrics to a local job scheduler when ``HEIMDALL_JOB_ID`` is set
    (``train.py:61-84``).  Never raises; does nothing without the variable."""
    job = os.environ.get("HEIMDALL_JOB_ID")
    if not job:
        return
    global _scheduler_client
    try:
        import httpx
        if _scheduler_client is None:
            _scheduler_client = httpx.Client(timeout=2.0)
        url = os.environ.get("HEIMDALL_URL", "http://localhost:7000")
        clean = {k: v for k, v in metrics.items() if v is not None}
        if clean:
            _scheduler_client.post(f"{url}/api/v1/jobs/{job}/metrics", json={"step": step, "metrics": clean})
    except Exception:                   # noqa: BLE001
        pass
