"""Parallelism: communication strategies, process groups, tensor parallelism."""
from __future__ import annotations

import logging

import torch.distributed as dist

from .comm import LibraryComm, LocalComm

logger = logging.getLogger(__name__)


def make_comm(backend: str = "auto", world: int | None = None, distributed_muon: bool = True):
    """``auto``: no-op for one rank, in-kernel NVLink collectives on CUDA when the symmetric
    memory layer is usable, library collectives otherwise."""
    if world is None:
        world = dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1
    if world == 1:
        return LocalComm()
    if backend in ("auto", "native"):
        try:
            from .native import NativeComm
            comm = NativeComm(distributed_muon=distributed_muon)
            logger.warning("communication: in-kernel NVLink collectives (NativeComm)")
            return comm
        except Exception as e:
            if backend == "native":
                raise
            logger.warning("communication: in-kernel collectives unavailable (%s: %s); "
                           "falling back to library collectives (LibraryComm)", type(e).__name__, e)
    return LibraryComm(distributed_muon=distributed_muon)


__all__ = ["make_comm", "LocalComm", "LibraryComm"]
