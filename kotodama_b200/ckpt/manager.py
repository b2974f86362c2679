"""Checkpointing: synchronous and asynchronous managers, SIGTERM flag, atomic files, rotation.

File format (loadable by the reference and vice versa, ``src/training/checkpoint.py:101-127``):
one ``torch.save`` pickle ``step_{step:08d}.pt`` (optionally ``.pt.zst``) holding ``step``,
``tokens_consumed``, ``model`` (state dict of the unwrapped model: separate q/k/v and gate/up
tensors whatever the executor's internal layout), ``muon_optimizer`` (torch optimizer layout +
``ns_coefficients``), ``adamw_optimizer``, ``scheduler`` (six scalars), optional ``data``, and
any ``extra`` keys merged at top level.

Asynchronous mode (``checkpoint.py:209-613``): the training thread pays only for a deep copy of
the state to host memory; a daemon thread writes to a shared-memory directory, compresses
(``zstd -3 -T0`` when the tool exists), copies atomically into the durable directory and rotates
both places.  Every file appears under its final name only by ``rename``.
"""
from __future__ import annotations

import hashlib
import logging
import os
import queue
import shutil
import signal
import subprocess
import threading
import time
from pathlib import Path
from typing import Any, Optional

import torch
import torch.distributed as dist

logger = logging.getLogger(__name__)


class SIGTERMHandler:
    """Sets ``received`` on SIGTERM; the loop checkpoints and leaves at the next step boundary."""

    def __init__(self) -> None:
        self.received = False
        self._previous = None
        try:
            self._previous = signal.signal(signal.SIGTERM, self._handle)
        except ValueError:          # not the main thread
            self._previous = None

    def _handle(self, signum: int, frame: Any) -> None:
        logger.warning("SIGTERM received: checkpoint at the next step boundary, then exit")
        self.received = True

    def restore(self) -> None:
        if self._previous is not None:
            signal.signal(signal.SIGTERM, self._previous)
            self._previous = None


def scheduler_state(scheduler: Any) -> dict[str, Any]:
    return {k: getattr(scheduler, k) for k in ("muon_base_lr", "adamw_base_lr", "warmup_steps", "total_steps",
                                               "decay_start_step", "decay_type")}


def unwrap_model(model: Any) -> Any:
    m = model.module if hasattr(model, "module") else model
    return m._orig_mod if hasattr(m, "_orig_mod") else m


def clean_state_dict(sd: dict[str, Any]) -> dict[str, Any]:
    """Drop wrapper prefixes left by ``torch.compile`` / DDP in foreign checkpoints."""
    return {k.replace("_orig_mod.", "").removeprefix("module."): v for k, v in sd.items()}


def _deep_cpu(obj: Any) -> Any:
    if isinstance(obj, torch.Tensor):
        return obj.detach().to("cpu", copy=True)
    if isinstance(obj, dict):
        return {k: _deep_cpu(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return type(obj)(_deep_cpu(v) for v in obj)
    return obj


def _world() -> int:
    return dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1


def _barrier() -> None:
    if _world() > 1:
        dist.barrier()


def zstd_available() -> bool:
    return shutil.which("zstd") is not None


def _atomic_save(state: dict[str, Any], path: Path) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    torch.save(state, tmp)
    os.replace(tmp, path)


def _step_of(p: Path) -> int:
    return int(p.name.split("_")[1].split(".")[0])


def list_checkpoints(d: Path) -> list[Path]:
    files = [p for p in d.glob("step_*.pt*") if p.name.endswith(".pt") or p.name.endswith(".pt.zst")]
    return sorted(files, key=lambda p: (_step_of(p), p.name.endswith(".zst")))


def load_checkpoint_file(path: Path, map_location: Any = "cpu") -> dict[str, Any]:
    if path.name.endswith(".zst"):
        if not zstd_available():
            raise RuntimeError(f"{path} is zstd-compressed and no `zstd` tool is installed")
        raw = subprocess.run(["zstd", "-d", "-c", str(path)], check=True, capture_output=True).stdout
        import io
        return torch.load(io.BytesIO(raw), map_location=map_location, weights_only=False)
    return torch.load(path, map_location=map_location, weights_only=False)


class CheckpointManager:
    """Rank 0 writes; every rank calls :meth:`save` (it ends with a barrier)."""

    def __init__(self, checkpoint_dir: str | Path, rank: int = 0, keep_last_n: int = 5) -> None:
        self.checkpoint_dir = Path(checkpoint_dir)
        self.rank = rank
        self.keep_last_n = keep_last_n
        if rank == 0:
            self.checkpoint_dir.mkdir(parents=True, exist_ok=True)

    # -- state assembly ------------------------------------------------------
    def _collect(self, step: int, model: Any, muon_opt: Any, adamw_opt: Any, scheduler: Any, tokens_consumed: int,
                 data_state: Optional[dict], extra: Optional[dict]) -> Optional[dict[str, Any]]:
        """Optimizer state may be spread over ranks (owner-computes Muon): assembling it is collective,
        so every rank runs this; only rank 0 keeps the result."""
        muon_sd = muon_opt.state_dict()
        adamw_sd = adamw_opt.state_dict()
        model_sd = unwrap_model(model).state_dict()
        gather = getattr(model, "_kotodama_gather_state", None) or getattr(unwrap_model(model), "_kotodama_gather_state", None)
        if gather is not None:                 # tensor-parallel shards -> full tensors
            model_sd = gather(model_sd)
        if self.rank != 0:
            return None
        # parameters may be views into one flat arena: store independent host tensors
        model_sd = {k: v.detach().to("cpu", copy=True) if isinstance(v, torch.Tensor) else v
                    for k, v in model_sd.items()}
        state = {"step": step, "tokens_consumed": tokens_consumed, "model": model_sd,
                 "muon_optimizer": muon_sd, "adamw_optimizer": adamw_sd, "scheduler": scheduler_state(scheduler)}
        if data_state is not None:
            state["data"] = data_state
        if extra:
            state.update(extra)
        return state

    def save(self, step: int, model: Any, muon_opt: Any, adamw_opt: Any, scheduler: Any, tokens_consumed: int = 0,
             data_state: Optional[dict] = None, extra: Optional[dict] = None) -> Optional[Path]:
        state = self._collect(step, model, muon_opt, adamw_opt, scheduler, tokens_consumed, data_state, extra)
        path = None
        if self.rank == 0:
            path = self.checkpoint_dir / f"step_{step:08d}.pt"
            t0 = time.time()
            _atomic_save(state, path)
            logger.info("Checkpoint saved: %s (%.1fs)", path, time.time() - t0)
            self._rotate(self.checkpoint_dir)
        _barrier()
        return path

    save_blocking = save

    def _rotate(self, d: Path) -> None:
        files = list_checkpoints(d)
        steps = sorted({_step_of(p) for p in files})
        for s in steps[:-self.keep_last_n] if self.keep_last_n > 0 else []:
            for p in files:
                if _step_of(p) == s:
                    try:
                        p.unlink()
                    except OSError as e:
                        logger.warning("Failed to remove %s: %s", p, e)

    # -- load -----------------------------------------------------------------
    def latest(self) -> Optional[Path]:
        if not self.checkpoint_dir.exists():
            return None
        files = list_checkpoints(self.checkpoint_dir)
        return files[-1] if files else None

    def load_latest(self, model: Any, muon_opt: Any, adamw_opt: Any, device: Any = "cpu") -> Optional[dict[str, Any]]:
        """Load the newest checkpoint into model and optimizers; returns its dict (without the big
        tensors' duplicates) or ``None`` when the directory has none.  A file that does not load
        (truncated, corrupt) is skipped with a warning and the next older one is tried."""
        if not self.checkpoint_dir.exists():
            return None
        for path in reversed(list_checkpoints(self.checkpoint_dir)):
            try:
                state = load_checkpoint_file(path, map_location="cpu")
            except Exception as e:          # noqa: BLE001 - any unreadable file is skipped
                logger.warning("Skipping unreadable checkpoint %s: %s", path, e)
                continue
            target = unwrap_model(model)
            sd = clean_state_dict(state["model"])
            scatter = getattr(target, "_kotodama_scatter_state", None)
            if scatter is not None:
                sd = scatter(sd)
            with torch.no_grad():
                own = target.state_dict()
                for k, v in sd.items():
                    if k in own:
                        own[k].copy_(v)
                missing = [k for k in own if k not in sd]
                if missing:
                    logger.warning("Checkpoint lacks %d keys, e.g. %s", len(missing), missing[:3])
            if state.get("muon_optimizer"):
                muon_opt.load_state_dict(state["muon_optimizer"])
            if state.get("adamw_optimizer"):
                adamw_opt.load_state_dict(state["adamw_optimizer"])
            logger.info("Resumed from %s (step %d)", path, state["step"])
            return state
        return None

    def shutdown(self) -> None:
        return None


_SHUTDOWN = object()


class AsyncCheckpointManager(CheckpointManager):
    """Host clone on the training thread, everything else on a daemon thread."""

    def __init__(self, checkpoint_dir: str | Path, rank: int = 0, keep_last_n: int = 5,
                 shm_dir: str | Path = "/dev/shm/luxia-base-ckpts", compress: bool = True,
                 queue_size: int = 5) -> None:
        super().__init__(checkpoint_dir, rank, keep_last_n)
        tag = hashlib.sha256(str(self.checkpoint_dir.resolve()).encode()).hexdigest()[:12]
        self.shm_dir = Path(shm_dir) / f"{self.checkpoint_dir.name}_{tag}"
        self.compress = compress and zstd_available()
        if compress and not self.compress and rank == 0:
            logger.warning("zstd tool not found: asynchronous checkpoints stay uncompressed")
        self._queue: "queue.Queue[Any]" = queue.Queue(maxsize=queue_size)
        self._worker: Optional[threading.Thread] = None
        self.errors: list[str] = []
        self.written: list[Path] = []
        if rank == 0:
            self.shm_dir.mkdir(parents=True, exist_ok=True)
            self._worker = threading.Thread(target=self._run, name="ckpt-writer", daemon=True)
            self._worker.start()

    def save(self, step: int, model: Any, muon_opt: Any, adamw_opt: Any, scheduler: Any, tokens_consumed: int = 0,
             data_state: Optional[dict] = None, extra: Optional[dict] = None) -> Optional[Path]:
        state = self._collect(step, model, muon_opt, adamw_opt, scheduler, tokens_consumed, data_state, extra)
        if self.rank == 0:
            t0 = time.time()
            state = _deep_cpu(state)
            logger.info("Checkpoint step %d cloned to host in %.2fs", step, time.time() - t0)
        _barrier()
        if self.rank == 0:
            if self._queue.full():
                logger.warning("Checkpoint queue full: step %d waits for the writer", step)
            self._queue.put((step, state))
            return self.checkpoint_dir / f"step_{step:08d}.pt"
        return None

    def save_blocking(self, *args: Any, **kw: Any) -> Optional[Path]:
        """Synchronous save on the calling thread (SIGTERM path: the writer may not get to finish)."""
        return CheckpointManager.save(self, *args, **kw)

    # -- worker -----------------------------------------------------------------
    def _run(self) -> None:
        while True:
            item = self._queue.get()
            try:
                if item is _SHUTDOWN:
                    return
                self._process(*item)
            except Exception as e:      # noqa: BLE001 - the training loop must not die for a failed save
                self.errors.append(f"{type(e).__name__}: {e}")
                logger.exception("Background checkpoint failed")
            finally:
                self._queue.task_done()

    def _write_shm(self, state: dict[str, Any], path: Path) -> None:
        _atomic_save(state, path)

    def _process(self, step: int, state: dict[str, Any]) -> None:
        shm_path = self.shm_dir / f"step_{step:08d}.pt"
        try:
            self._write_shm(state, shm_path)
        except Exception:
            for p in (shm_path, shm_path.with_suffix(".pt.tmp")):
                p.unlink(missing_ok=True)
            raise
        final = shm_path
        if self.compress and self._queue.qsize() <= 2:      # under backpressure keep the raw file
            zst = shm_path.with_suffix(".pt.zst")
            tmp = zst.with_suffix(".zst.tmp")
            r = subprocess.run(["zstd", "-3", "-T0", "-q", "-f", str(shm_path), "-o", str(tmp)], capture_output=True)
            if r.returncode == 0:
                os.replace(tmp, zst)
                shm_path.unlink(missing_ok=True)
                final = zst
            else:
                tmp.unlink(missing_ok=True)
                logger.warning("zstd failed (%s): keeping uncompressed checkpoint", r.stderr.decode()[:200])
        try:
            self._persist(final)
        except OSError as e:
            self.errors.append(f"persist: {e}")
            logger.error("Could not persist %s (%s): the shared-memory copy is kept", final, e)
            return
        self._rotate(self.shm_dir)
        self._rotate(self.checkpoint_dir)

    def _persist(self, src: Path) -> None:
        dst = self.checkpoint_dir / src.name
        tmp = dst.with_suffix(dst.suffix + ".tmp")
        shutil.copy2(src, tmp)
        os.replace(tmp, dst)
        self.written.append(dst)

    def wait(self) -> None:
        """Block until everything queued so far has been written."""
        if self._worker is not None:
            self._queue.join()

    def shutdown(self, timeout: float = 120.0) -> None:
        if self._worker is None:
            return
        self._queue.put(_SHUTDOWN)
        self._worker.join(timeout)
        if self._worker.is_alive():
            logger.error("Checkpoint writer still busy after %.0fs", timeout)
        self._worker = None
