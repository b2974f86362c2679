"""Causal GQA attention for the CUDA backend.

Inference (prefill, evaluation) runs the tcgen05 flash-attention forward in
``csrc/attn_sm100.cu`` when the shape is one it covers (head_dim 128, sequence length a multiple
of 128).  The training path needs a backward as well; until the native one lands it uses PyTorch's
fused scaled-dot-product attention for both directions (a library kernel, reported as such by
``CudaOps.attention_library_calls``); ``KOTODAMA_FLASH_TRAIN=1`` switches training to the native
forward with the ``flash_attn`` library's backward.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def _native_ok(ops, q: torch.Tensor, need_grad: bool) -> bool:
    from .flash import supported
    if not getattr(ops, "native_attention", True) or not supported(q):
        return False
    # training keeps forward and backward in one library call pair unless asked otherwise
    return (not need_grad) or getattr(ops, "native_attention_train", False)


def attention_fwd(ops, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, need_grad: bool = True):
    if _native_ok(ops, q, need_grad):
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
