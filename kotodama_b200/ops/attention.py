"""Causal GQA attention for the CUDA backend.

Dispatches to the tcgen05 flash-attention kernels in ``csrc/attn_sm100.cu`` when the shape
is one they cover (head_dim 128 or 64, sequence length a multiple of the tile); any other
shape goes to PyTorch's fused scaled-dot-product attention, which is a library kernel and is
reported as such by ``CudaOps.attention_library_calls``.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _native_ok(ops, q: torch.Tensor) -> bool:
    return getattr(ops, "native_attention", False) and q.shape[-1] in (64, 128) and q.shape[1] % 128 == 0


def attention_fwd(ops, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, need_grad: bool = True):
    if _native_ok(ops, q):
        from .flash import flash_fwd
        return flash_fwd(ops, q, k, v)
    ops.attention_library_calls = getattr(ops, "attention_library_calls", 0) + 1
    if not need_grad:
        o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=True,
                                           enable_gqa=q.shape[2] != k.shape[2])
        return o.transpose(1, 2).contiguous(), None
    with torch.enable_grad():
        ql = q.detach().transpose(1, 2).requires_grad_(True)
        kl = k.detach().transpose(1, 2).requires_grad_(True)
        vl = v.detach().transpose(1, 2).requires_grad_(True)
        o = F.scaled_dot_product_attention(ql, kl, vl, is_causal=True, enable_gqa=ql.shape[1] != kl.shape[1])
    out = o.detach().transpose(1, 2).contiguous()
    return out, (o, ql, kl, vl)


def attention_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out) -> None:
    if not isinstance(lse, tuple):
        from .flash import flash_bwd
        return flash_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out)
    og, ql, kl, vl = lse
    dq, dk, dv = torch.autograd.grad(og, (ql, kl, vl), do.transpose(1, 2))
    dq_out.copy_(dq.transpose(1, 2))
    dk_out.copy_(dk.transpose(1, 2))
    dv_out.copy_(dv.transpose(1, 2))
