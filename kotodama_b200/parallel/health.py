"""Host-side peer health over the rendezvous store: who is alive, who has left.

The reference has no rank-failure detection (``src/training/train.py`` only reacts to SIGTERM on
its own process).  Here every rank writes a heartbeat (its current step) into the process group's
key-value store once per step and, before it launches the next step's kernels and collectives,
looks for departure notices of its peers.  A rank that stops between steps (exception, SIGTERM
drain, operator stop) announces it; the others then raise on the host instead of entering a
collective that can no longer complete.  Nothing here touches the GPU, so it also works when a
device has stopped answering.  A rank that dies without a notice is still caught by the process
group's collective timeout; ``stale()`` names the ranks whose heartbeat has not moved.
"""
from __future__ import annotations

import time
from typing import Any, Optional

import torch.distributed as dist


class PeerLeft(RuntimeError):
    """Raised on a surviving rank when a peer has announced that it is leaving the job."""


class PeerHealth:
    def __init__(self, store: Any = None, rank: Optional[int] = None, world: Optional[int] = None,
                 prefix: str = "kotodama/health") -> None:
        if store is None:
            store = dist.distributed_c10d._get_default_store()
        self.store = store
        self.rank = dist.get_rank() if rank is None else rank
        self.world = dist.get_world_size() if world is None else world
        self.prefix = prefix
        self._seen: dict[int, tuple[str, float]] = {}

    def _key(self, kind: str, rank: int) -> str:
        return f"{self.prefix}/{kind}/{rank}"

    def beat(self, step: int) -> None:
        self.store.set(self._key("beat", self.rank), str(step))

    def announce_leave(self, reason: str = "") -> None:
        """Call on the way out, between steps, with none of this rank's kernels or collectives in flight."""
        try:
            self.store.set(self._key("left", self.rank), reason or "left")
        except Exception:                      # noqa: BLE001 - the store may already be gone
            pass

    def departed(self) -> dict[int, str]:
        """Ranks that have announced their departure (non-blocking)."""
        out = {}
        for r in range(self.world):
            if r != self.rank and self.store.check([self._key("left", r)]):
                out[r] = self.store.get(self._key("left", r)).decode()
        return out

    def raise_if_peer_left(self) -> None:
        gone = self.departed()
        if gone:
            raise PeerLeft(f"rank {self.rank}: peer rank(s) {sorted(gone)} left the job: {gone}")

    def stale(self, older_than_s: float) -> list[int]:
        """Ranks whose heartbeat value has not changed for ``older_than_s`` seconds (as seen from here)."""
        now = time.monotonic()
        out = []
        for r in range(self.world):
            if r == self.rank:
                continue
            k = self._key("beat", r)
            val = self.store.get(k).decode() if self.store.check([k]) else ""
            prev = self._seen.get(r)
            if prev is None or prev[0] != val:
                self._seen[r] = (val, now)
            elif now - prev[1] > older_than_s:
                out.append(r)
        return out
