"""Parallelism: communication strategies, process groups, tensor parallelism."""
from __future__ import annotations

import torch.distributed as dist

from .comm import LibraryComm, LocalComm


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
            return NativeComm(distributed_muon=distributed_muon)
        except Exception:
            if backend == "native":
                raise
    return LibraryComm(distributed_muon=distributed_muon)


__all__ = ["make_comm", "LocalComm", "LibraryComm"]
