"""Communication strategies used by the training executor.

The executor calls a small set of hooks (gradient ready per layer, gradient reduce finish,
global norm, parameter publish, tensor-parallel linear helpers); a strategy object decides
how they are carried out:

* :class:`LocalComm` — one rank, nothing to do.
* :class:`LibraryComm` — ``torch.distributed`` collectives (gloo on CPU, NCCL on GPU).  This
  is the measured baseline for the native path and the backend of CPU/gloo runs.  Gradients
  are averaged with per-layer asynchronous all-reduces launched while backward continues;
  with ``distributed_muon`` each matrix is orthogonalised only on its owner rank and the new
  parameter is broadcast from there.
* ``NativeComm`` (``kotodama_b200.parallel.native``) — the same schedule with in-kernel
  NVLink loads/stores on symmetric memory.

What the reference does at these points: stock DDP bucketed all-reduce
(``src/training/train.py:328-340``) and Newton-Schulz replicated on every rank
(``src/training/muon.py:255-351``).
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist


def _fp8_kw(w: Any) -> dict:
    """Weight gradients follow the precision of their weight: fp8 when the weight is an ``Fp8Weight``."""
    return {} if isinstance(w, torch.Tensor) else {"fp8": True}


class LocalComm:
    world = 1
    rank = 0
    dp_size = 1
    tp_size = 1
    distributed_muon = False

    def allocator(self, device: torch.device, dtype: torch.dtype):
        return lambda n: torch.zeros(n, device=device, dtype=dtype)

    def attach(self, engine: Any) -> None:
        self.engine = engine

    # tensor-parallel helpers (identity without TP)
    def sp_gather(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def shard_tokens(self, x: torch.Tensor) -> torch.Tensor:
        return x

    def loss_reduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of per-rank loss terms / token counts over the ranks that split one batch."""
        return t

    def runs_ns(self, slot) -> bool:
        return True

    def row_linear(self, ops, x, w, residual=None):
        return ops.gemm_nt(x, w, residual=residual)

    def row_linear_bwd_input(self, ops, dy, w):
        return ops.gemm_nn(dy, w)

    def col_linear_bwd_input(self, ops, dy, w):
        return ops.gemm_nn(dy, w)

    # Composite hooks the executor calls; strategies with fused GEMM+collective kernels override
    # these, everything else inherits the compositions of the primitive hooks above.
    def col_linear(self, ops, x, w):
        """Column-parallel projection of a sequence-sharded activation: all-gather -> GEMM."""
        return ops.gemm_nt(self.sp_gather(x), w)

    def row_linear_bwd(self, ops, dy, w, x_saved, g_out, accumulate: bool):
        """Backward of a row-parallel projection: all-gather(dy) -> data gradient and weight gradient."""
        dyg = self.sp_gather(dy)
        dx = ops.gemm_nn(dyg, w)
        ops.gemm_tn(dyg, x_saved, out=g_out, accumulate=accumulate, **_fp8_kw(w))
        return dx

    def col_linear_bwd(self, ops, dy, w, x, g_out, accumulate: bool):
        """Backward of a column-parallel projection: weight gradient from the re-gathered input,
        data gradient GEMM -> reduce-scatter."""
        ops.gemm_tn(dy, self.sp_gather(x), out=g_out, accumulate=accumulate, **_fp8_kw(w))
        return self.col_linear_bwd_input(ops, dy, w)

    # gradient reduction
    def layer_grads_ready(self, layer: int) -> None:
        pass

    def small_grads_ready(self) -> None:
        pass

    def finish_grad_reduce(self) -> None:
        pass

    def grad_sumsq(self, ops) -> torch.Tensor:
        return ops.sumsq(self.engine.arena.grads)

    # Muon
    def full_shape(self, slot) -> tuple[int, int]:
        return slot.shape

    def muon_gather(self, slot, x):
        return x

    def muon_scatter(self, slot, x, transposed: bool):
        return x

    def muon_apply(self, ops, slot, orth, lr: float, wd: float, scale: float, transposed: bool) -> None:
        """Write the Muon update of one matrix (strategies that own the write may also publish it)."""
        ops.muon_apply(self.engine.arena.view(slot.name), orth, lr, wd, scale, transposed)

    def finish_param_publish(self) -> None:
        pass

    def gather_momentum(self, slot, buf):
        return buf

    def shard_like(self, slot, full):
        return full

    def barrier(self) -> None:
        pass

    def all_reduce_max(self, value: float) -> float:
        return value


class LibraryComm(LocalComm):
    """Data-parallel strategy on ``torch.distributed`` collectives."""

    def __init__(self, group: Optional[dist.ProcessGroup] = None, distributed_muon: bool = True) -> None:
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        self.dp_size = self.world
        self.distributed_muon = distributed_muon and self.world > 1
        self._pending: list = []

    def attach(self, engine: Any) -> None:
        self.engine = engine
        ar = engine.arena
        # every rank starts from rank 0's weights (DDP constructor broadcast, ``train.py:332-337``)
        dist.broadcast(ar.params, src=self._global(0), group=self.group)
        self._layer_ranges: dict[int, tuple[int, int]] = {}
        for s in ar.muon_slots():
            lo, hi = self._layer_ranges.get(s.layer, (s.offset, s.offset + s.numel))
            self._layer_ranges[s.layer] = (min(lo, s.offset), max(hi, s.offset + s.numel))

    def _global(self, group_rank: int) -> int:
        return dist.get_global_rank(self.group, group_rank) if self.group is not None else group_rank

    def _reduce_range(self, lo: int, hi: int) -> None:
        g = self.engine.arena.grads[lo:hi]
        # c10d orders the collective after the kernels already queued on the current stream
        self._pending.append(dist.all_reduce(g, op=dist.ReduceOp.SUM, group=self.group, async_op=True))

    def layer_grads_ready(self, layer: int) -> None:
        lo, hi = self._layer_ranges[layer]
        self._reduce_range(lo, hi)

    def small_grads_ready(self) -> None:
        ar = self.engine.arena
        lo, hi = ar.adamw_range()
        self._reduce_range(lo, hi)
        if -1 in self._layer_ranges:
            self._reduce_range(*self._layer_ranges[-1])

    def finish_grad_reduce(self) -> None:
        for w in self._pending:
            w.wait()
        self._pending.clear()

    def finish_param_publish(self) -> None:
        if not self.distributed_muon:
            return
        ar = self.engine.arena
        works = []
        for s in ar.muon_slots():
            works.append(dist.broadcast(ar.view(s.name), src=self._global(s.owner), group=self.group, async_op=True))
        for w in works:
            w.wait()

    def gather_momentum(self, slot, buf):
        """Momentum lives on the owner only; checkpoints need it on rank 0 in the full layout."""
        if not self.distributed_muon:
            return buf
        if buf is None:
            buf = torch.zeros(slot.shape, device=self.engine.device, dtype=self.engine.dtype)
        out = buf.clone()
        dist.broadcast(out, src=self._global(slot.owner), group=self.group)
        return out

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def all_reduce_max(self, value: float) -> float:
        dev = self.engine.device if hasattr(self, "engine") else "cpu"
        t = torch.tensor([value], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
