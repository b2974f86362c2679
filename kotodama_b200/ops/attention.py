"""Causal GQA attention for the CUDA backend: the tcgen05 flash-attention kernels in both
directions (``ops/flash.py``).  There is no library attention on this backend; a shape the kernels
do not cover (head_dim other than 64 / 128, a dtype other than bf16) raises."""
from __future__ import annotations

import torch

from .flash import flash_bwd, flash_fwd, supported


def attention_fwd(ops, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, need_grad: bool = True,
                  cu_seqlens=None, max_seqlen: int = 0):
    if not supported(q):
        raise NotImplementedError(f"native attention covers bf16 with head_dim 64 or 128, got {q.dtype} {tuple(q.shape)}")
    return flash_fwd(ops, q, k, v, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)


def attention_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out) -> None:
    flash_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out)
