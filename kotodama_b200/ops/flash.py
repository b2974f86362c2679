"""Python side of the tcgen05 flash-attention kernels (``csrc/attn_sm100.cu``).

Forward: causal GQA attention for head_dim 128 and sequence lengths that are multiples of 128,
reading q / k / v straight out of the fused projection buffers (token-major rows, heads side by
side, any row stride).  Backward of the training path is taken from the ``flash_attn`` library
(given our forward's output and log-sum-exp) until the native backward lands; that call is
counted in ``attention_library_calls``.
"""
from __future__ import annotations

import ctypes
import math

import torch

_VP, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def supported(q: torch.Tensor) -> bool:
    return (q.is_cuda and q.dtype == torch.bfloat16 and q.ndim == 4 and q.shape[-1] == 128
            and q.stride(-1) == 1 and q.stride(2) == 128 and q.stride(0) == q.shape[1] * q.stride(1))


def flash_fwd(ops, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor):
    """``q[B,T,H,128]``, ``k,v[B,T,KV,128]`` (views with a token stride) -> ``o[B,T,H,128]``, ``lse[B,H,T]``."""
    B, T, H, hd = q.shape
    KV = k.shape[2]
    o = torch.empty(B, T, H, hd, device=q.device, dtype=q.dtype)
    lse = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    st = _VP(torch.cuda.current_stream().cuda_stream)
    rc = ops.lib.kb_flash_fwd(_VP(q.data_ptr()), _LL(q.stride(1)), _I(H * hd), _I(0),
                              _VP(k.data_ptr()), _LL(k.stride(1)), _I(KV * hd), _I(0),
                              _VP(v.data_ptr()), _LL(v.stride(1)), _I(KV * hd), _I(0),
                              _VP(o.data_ptr()), _VP(lse.data_ptr()), _I(B), _I(T), _I(H), _I(KV), _I(hd),
                              _F(1.0 / math.sqrt(hd)), _VP(ops.status(q.device).data_ptr()), st)
    ops._rc(rc, "kb_flash_fwd")
    return o, lse


def flash_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out) -> None:
    from flash_attn.flash_attn_interface import _flash_attn_backward
    ops.attention_library_calls = getattr(ops, "attention_library_calls", 0) + 1
    B, T, H, hd = q.shape
    dq = torch.empty(B, T, H, hd, device=q.device, dtype=q.dtype)
    dk = torch.empty(B, T, k.shape[2], hd, device=q.device, dtype=q.dtype)
    dv = torch.empty_like(dk)
    _flash_attn_backward(do.contiguous(), q, k, v, o, lse, dq, dk, dv, 0.0, 1.0 / math.sqrt(hd), True, -1, 0, 0.0,
                         None, False, None)
    dq_out.copy_(dq)
    dk_out.copy_(dk)
    dv_out.copy_(dv)
