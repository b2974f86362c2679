"""Tensor parallelism.

Two layers:

1. The reference's API for autograd models (``src/training/tensor_parallel.py``): conjugate
   copy / reduce operators (``:31-75``), contiguous TP groups with strided DP groups
   (``:81-116``), in-place sharding of plain ``nn.Linear`` weights with ``_tp_*`` tags
   (``:189-254``), all-gather along a dim (``:260-272``), QK-norm gradient sum (``:278-295``)
   and TP-aware clipping (``:298-330``).

2. :class:`TensorParallelComm`, the strategy the training executor uses for TP with
   sequence parallelism: tokens are sharded over the TP ranks for routing, norms, residuals and
   the loss head; activations are all-gathered in front of the column-parallel GEMMs and
   reduce-scattered behind the row-parallel ones; Muon gathers each matrix to one owner rank,
   orthogonalises it there and returns the shards (the reference runs the full Newton-Schulz on
   every TP rank, ``src/training/muon.py:286-296``).
"""
from __future__ import annotations

from typing import Any, Optional

import torch
import torch.distributed as dist
import torch.nn as nn

from .comm import LocalComm


# --------------------------------------------------------------------------- autograd operators
class _CopyToParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        ctx.group = group
        return x

    @staticmethod
    def backward(ctx, g):
        g = g.contiguous()
        dist.all_reduce(g, group=ctx.group)
        return g, None


class _ReduceFromParallelRegion(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, group):
        x = x.contiguous().clone()
        dist.all_reduce(x, group=group)
        return x

    @staticmethod
    def backward(ctx, g):
        return g, None


def copy_to_parallel_region(x: torch.Tensor, group: Any) -> torch.Tensor:
    return _CopyToParallelRegion.apply(x, group)


def reduce_from_parallel_region(x: torch.Tensor, group: Any) -> torch.Tensor:
    return _ReduceFromParallelRegion.apply(x, group)


def all_gather_along_dim(x: torch.Tensor, dim: int, group: Any) -> torch.Tensor:
    parts = [torch.empty_like(x) for _ in range(dist.get_world_size(group))]
    dist.all_gather(parts, x.contiguous(), group=group)
    return torch.cat(parts, dim=dim)


# --------------------------------------------------------------------------- groups
def create_process_groups(world_size: int, tp_size: int) -> tuple[Any, Any]:
    """TP groups are runs of ``tp_size`` consecutive ranks; DP groups take every ``tp_size``-th rank.
    Every rank must call this (``new_group`` is collective).  Returns this rank's (tp, dp) groups."""
    if world_size % tp_size:
        raise ValueError(f"world_size {world_size} is not a multiple of tp_size {tp_size}")
    rank = dist.get_rank()
    tp_group = dp_group = None
    for start in range(0, world_size, tp_size):
        ranks = list(range(start, start + tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            tp_group = g
    for off in range(tp_size):
        ranks = list(range(off, world_size, tp_size))
        g = dist.new_group(ranks)
        if rank in ranks:
            dp_group = g
    return tp_group, dp_group


COLUMN_PARALLEL = ("q_proj", "k_proj", "v_proj", "gate_proj", "up_proj")   # shard dim 0 (outputs)
ROW_PARALLEL = ("o_proj", "down_proj")                                     # shard dim 1 (inputs)


def shard_dim_of(name: str) -> Optional[int]:
    if any(k in name for k in COLUMN_PARALLEL):
        return 0
    if any(k in name for k in ROW_PARALLEL):
        return 1
    return None


def apply_tensor_parallelism(model: nn.Module, tp_group: Any) -> None:
    """Shard projection weights in place and tag them; embeddings, LM head, norms and AttnRes
    parameters stay replicated."""
    size, rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
    cfg = model.config
    if cfg.num_attention_heads % size or cfg.num_kv_heads % size or cfg.intermediate_size % size:
        raise ValueError("heads / kv heads / FFN width must divide by tp_size")
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear):
            d = shard_dim_of(name)
            if d is None:
                continue
            n = mod.weight.shape[d] // size
            shard = mod.weight.data.narrow(d, rank * n, n).contiguous()
            mod.weight = nn.Parameter(shard)
            for k, v in (("_tp_shard_dim", d), ("_tp_group", tp_group), ("_tp_size", size), ("_tp_rank", rank)):
                setattr(mod.weight, k, v)
            if d == 0:
                mod.out_features = n
            else:
                mod.in_features = n
    for layer in model.layers:
        layer.attn.tp_group = tp_group
        layer.ffn.tp_group = tp_group
        layer.attn.num_heads = cfg.num_attention_heads // size
        layer.attn.num_kv_heads = cfg.num_kv_heads // size


def gather_full_state_dict(model: nn.Module, tp_group: Any) -> dict[str, torch.Tensor]:
    """Checkpoint view under TP: sharded weights are gathered to full tensors so the file has the
    same layout as a data-parallel run (the reference writes rank 0's shard only,
    ``src/training/checkpoint.py:101-112``)."""
    out = {}
    params = dict(model.named_parameters())
    for k, v in model.state_dict().items():
        p = params.get(k)
        d = getattr(p, "_tp_shard_dim", None) if p is not None else None
        out[k] = all_gather_along_dim(v.detach(), d, tp_group) if d is not None else v.detach()
    return out


def sync_tp_replicated_grads(model: nn.Module, tp_group: Any) -> None:
    """QK-norm weights see only the local heads: their gradients are summed over the TP group."""
    for name, p in model.named_parameters():
        if ("q_norm" in name or "k_norm" in name) and p.grad is not None:
            dist.all_reduce(p.grad, group=tp_group)


def tp_clip_grad_norm(model: nn.Module, max_norm: float, tp_group: Any) -> torch.Tensor:
    """Global-norm clip where sharded parameters contribute the sum over shards."""
    params = [p for p in (model.parameters() if isinstance(model, nn.Module) else model) if p.grad is not None]
    dev = params[0].grad.device if params else torch.device("cpu")
    sharded = torch.zeros((), device=dev)
    replicated = torch.zeros((), device=dev)
    for p in params:
        sq = p.grad.float().pow(2).sum()
        if hasattr(p, "_tp_shard_dim"):
            sharded = sharded + sq
        else:
            replicated = replicated + sq
    dist.all_reduce(sharded, group=tp_group)
    total = (sharded + replicated).sqrt()
    coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
    for p in params:
        p.grad.mul_(coef.to(p.grad.dtype))
    return total


# --------------------------------------------------------------------------- executor strategy
class TensorParallelComm(LocalComm):
    """TP (+ optional DP) with sequence parallelism for the hand-scheduled executor."""

    def __init__(self, tp_group: Any, dp_group: Any = None, sequence_parallel: bool = True) -> None:
        self.tp_group, self.dp_group = tp_group, dp_group
        self.tp_size, self.tp_rank = dist.get_world_size(tp_group), dist.get_rank(tp_group)
        self.dp_size = dist.get_world_size(dp_group) if dp_group is not None else 1
        self.dp_rank = dist.get_rank(dp_group) if dp_group is not None else 0
        self.world, self.rank = self.dp_size, self.dp_rank       # "world" of the gradient reduction = DP
        self.sequence_parallel = sequence_parallel
        self.distributed_muon = False

    # ---- model preparation -------------------------------------------------
    def prepare_model(self, model: nn.Module) -> None:
        if not any(hasattr(p, "_tp_shard_dim") for p in model.parameters()):
            apply_tensor_parallelism(model, self.tp_group)
        model._kotodama_gather_state = lambda sd: gather_full_state_dict(model, self.tp_group)
        model._kotodama_scatter_state = self._scatter_state
        self._model = model

    def _scatter_state(self, sd: dict[str, torch.Tensor]) -> dict[str, torch.Tensor]:
        out = {}
        for k, v in sd.items():
            d = shard_dim_of(k) if k.endswith("weight") and v.ndim == 2 else None
            if d is not None:
                n = v.shape[d] // self.tp_size
                v = v.narrow(d, self.tp_rank * n, n)
            out[k] = v
        return out

    def attach(self, engine: Any) -> None:
        self.engine = engine
        src = dist.get_global_rank(self.tp_group, 0)
        ar = engine.arena
        # replicated parameters must start identical inside the TP group; shards come from the same
        # full tensor on every rank (same seed), so a broadcast of the replicated range is enough
        lo, hi = ar.adamw_range()
        dist.broadcast(ar.params[lo:hi], src=src, group=self.tp_group)
        if self.dp_group is not None and self.dp_size > 1:
            dist.broadcast(ar.params, src=dist.get_global_rank(self.dp_group, 0), group=self.dp_group)

    # ---- sequence-parallel activations --------------------------------------
    def shard_tokens(self, x: torch.Tensor) -> torch.Tensor:
        if not self.sequence_parallel:
            return x
        n = x.shape[0] // self.tp_size
        return x[self.tp_rank * n:(self.tp_rank + 1) * n]

    def sp_gather(self, x: torch.Tensor) -> torch.Tensor:
        if not self.sequence_parallel:
            return x
        out = torch.empty(x.shape[0] * self.tp_size, *x.shape[1:], device=x.device, dtype=x.dtype)
        dist.all_gather_into_tensor(out, x.contiguous(), group=self.tp_group)
        return out

    def _reduce_scatter(self, full: torch.Tensor) -> torch.Tensor:
        if not self.sequence_parallel:
            dist.all_reduce(full, group=self.tp_group)
            return full
        out = torch.empty(full.shape[0] // self.tp_size, *full.shape[1:], device=full.device, dtype=full.dtype)
        dist.reduce_scatter_tensor(out, full.contiguous(), group=self.tp_group)
        return out

    def row_linear(self, ops, x, w, residual=None):
        y = self._reduce_scatter(ops.gemm_nt(x, w))
        if residual is not None:
            y = y + residual
        return y

    def row_linear_bwd_input(self, ops, dy, w):
        return ops.gemm_nn(self.sp_gather(dy), w)

    def col_linear_bwd_input(self, ops, dy, w):
        return self._reduce_scatter(ops.gemm_nn(dy, w))

    # ---- gradients ---------------------------------------------------------------
    def finish_grad_reduce(self) -> None:
        ar = self.engine.arena
        lo, hi = ar.adamw_range()
        # replicated parameters: each TP rank saw a different token shard (or different heads)
        if self.sequence_parallel:
            dist.all_reduce(ar.grads[lo:hi], group=self.tp_group)
        else:
            for s in ar.slots:
                if "q_norm" in s.name or "k_norm" in s.name:
                    dist.all_reduce(ar.view(s.name, grads=True), group=self.tp_group)
        if self.dp_group is not None and self.dp_size > 1:
            dist.all_reduce(ar.grads, group=self.dp_group)

    def grad_sumsq(self, ops) -> torch.Tensor:
        ar = self.engine.arena
        sharded = ops.sumsq(ar.grads[:ar.muon_end]).reshape(1).clone()
        dist.all_reduce(sharded, group=self.tp_group)
        lo, hi = ar.adamw_range()
        return (sharded + ops.sumsq(ar.grads[lo:hi]).reshape(1))[0]

    # ---- Muon ---------------------------------------------------------------------
    def full_shape(self, slot) -> tuple[int, int]:
        d = shard_dim_of(slot.name)
        shape = list(slot.shape)
        shape[d] *= self.tp_size
        return tuple(shape)

    def ns_owner(self, slot) -> int:
        return self.engine.arena.muon_slots().index(slot) % self.tp_size

    def runs_ns(self, slot) -> bool:
        return self.ns_owner(slot) == self.tp_rank

    def muon_gather(self, slot, x):
        return all_gather_along_dim(x, shard_dim_of(slot.name), self.tp_group)

    def muon_scatter(self, slot, x, transposed: bool):
        """Owner's orthogonalised matrix -> this rank's shard (in the parameter's own orientation)."""
        full = x.t().contiguous() if (transposed and self.runs_ns(slot)) else x
        rows, cols = self.full_shape(slot)
        if not self.runs_ns(slot):
            full = torch.empty(rows, cols, device=x.device, dtype=x.dtype)
        dist.broadcast(full, src=dist.get_global_rank(self.tp_group, self.ns_owner(slot)), group=self.tp_group)
        d = shard_dim_of(slot.name)
        n = slot.shape[d]
        return full.narrow(d, self.tp_rank * n, n).contiguous()

    def muon_exchange_group(self, slots, shards, orthogonalise):
        """Owner-computes Newton-Schulz for a group of same-shape, same-shard-dimension matrices with two
        collectives in total: an all-to-all that brings every shard of matrix ``i`` to rank ``i % tp`` (so
        each owner holds whole matrices and can orthogonalise them as one batch), and an all-to-all that
        returns to every rank its own shard of every result.  ``shards``: this rank's shard of each
        matrix, in ``slots`` order; ``orthogonalise(batch[n, rows, cols]) -> batch``.  Returns the
        orthogonalised shards in ``slots`` order.  (The reference gathers every matrix on every rank,
        one call per matrix, and repeats the iteration everywhere: ``muon.py:286-296``.)"""
        W, me = self.tp_size, self.tp_rank
        n = len(slots)
        d = shard_dim_of(slots[0].name)
        sr, sc = shards[0].shape
        numel = sr * sc
        owned_by = [[i for i in range(n) if i % W == o] for o in range(W)]
        n_me = len(owned_by[me])
        send = torch.cat([torch.stack([shards[i] for i in owned_by[o]]).reshape(-1) if owned_by[o]
                          else shards[0].new_empty(0) for o in range(W)])
        recv = send.new_empty(W * n_me * numel)
        dist.all_to_all_single(recv, send, output_split_sizes=[n_me * numel] * W,
                               input_split_sizes=[len(owned_by[o]) * numel for o in range(W)], group=self.tp_group)
        back_send = send.new_empty(W * n_me * numel)
        if n_me:
            parts = recv.view(W, n_me, sr, sc)
            full = (parts.permute(1, 0, 2, 3).reshape(n_me, W * sr, sc) if d == 0
                    else parts.permute(1, 2, 0, 3).reshape(n_me, sr, W * sc)).contiguous()
            orth = orthogonalise(full)
            out = (orth.reshape(n_me, W, sr, sc).permute(1, 0, 2, 3) if d == 0
                   else orth.reshape(n_me, sr, W, sc).permute(2, 0, 1, 3))
            back_send.view(W, n_me, sr, sc).copy_(out)
        back = send.new_empty(n * numel)
        dist.all_to_all_single(back, back_send, output_split_sizes=[len(owned_by[o]) * numel for o in range(W)],
                               input_split_sizes=[n_me * numel] * W, group=self.tp_group)
        res = [None] * n
        at = 0
        for o in range(W):
            for i in owned_by[o]:
                res[i] = back[at:at + numel].view(sr, sc)
                at += numel
        return res

    def gather_momentum(self, slot, buf):
        return all_gather_along_dim(buf, shard_dim_of(slot.name), self.tp_group)

    def shard_like(self, slot, full):
        d = shard_dim_of(slot.name)
        n = slot.shape[d]
        return full.narrow(d, self.tp_rank * n, n)

    def all_reduce_max(self, value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64, device=self.engine.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def loss_reduce(self, t: torch.Tensor) -> torch.Tensor:
        if self.sequence_parallel:
            dist.all_reduce(t, group=self.tp_group)
        return t
