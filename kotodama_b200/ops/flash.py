"""Python side of the tcgen05 flash-attention kernels (``csrc/attn_sm100.cu``, ``csrc/attn_bwd_sm100.cu``).

Causal GQA attention, forward and backward, for head_dim 64 / 128 and any sequence length, reading
q / k / v straight out of the fused projection buffers (token-major rows, heads side by side, any
row stride) and writing dq / dk / dv straight into the fused gradient buffers.  The forward also
takes packed variable-length sequences (``cu_seqlens``), which the serving engine uses for prefill.
Takes the place of the reference's FA2 / FA4 / SDPA dispatch (``src/model/llama.py:274-377``).
"""
from __future__ import annotations

import ctypes
import math
from typing import Optional

import torch

_VP, _I, _LL, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float


def _rows(x: torch.Tensor) -> tuple[int, int]:
    """(token stride, head stride check) of a ``[B, T, h, hd]`` view whose tokens are evenly spaced rows."""
    B, T, h, hd = x.shape
    if x.stride(-1) != 1 or x.stride(2) != hd or (B > 1 and x.stride(0) != T * x.stride(1)):
        raise ValueError(f"attention operand is not a token-major view: shape {tuple(x.shape)} strides {x.stride()}")
    return x.stride(1), h * hd


def supported(q: torch.Tensor) -> bool:
    return q.is_cuda and q.dtype == torch.bfloat16 and q.ndim == 4 and q.shape[-1] in (64, 128)


def flash_fwd(ops, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, cu_seqlens: Optional[torch.Tensor] = None,
              max_seqlen: int = 0):
    """``q[B,T,H,hd]``, ``k,v[B,T,KV,hd]`` (views with a token stride) -> ``o[B,T,H,hd]``, ``lse[B,H,T]``.

    Packed form: ``q[1,total,H,hd]`` etc. with ``cu_seqlens[n+1]`` (int32, device) and ``max_seqlen``;
    ``lse`` is then ``[H, total]``."""
    B, T, H, hd = q.shape
    KV = k.shape[2]
    qs, qc = _rows(q)
    ks, kc = _rows(k)
    vs, vc = _rows(v)
    o = torch.empty(B, T, H, hd, device=q.device, dtype=q.dtype)
    if cu_seqlens is not None:
        if B != 1:
            raise ValueError("packed attention takes q[1, total, H, hd]")
        nseq, total, max_t = cu_seqlens.numel() - 1, T, int(max_seqlen)
        lse = torch.empty(H, total, device=q.device, dtype=torch.float32)
        cu = _VP(cu_seqlens.data_ptr())
    else:
        nseq, total, max_t = B, B * T, T
        lse = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
        cu = _VP(0)
    st = _VP(torch.cuda.current_stream().cuda_stream)
    rc = ops.lib.kb_flash_fwd(_VP(q.data_ptr()), _LL(qs), _I(qc), _I(0), _VP(k.data_ptr()), _LL(ks), _I(kc), _I(0),
                              _VP(v.data_ptr()), _LL(vs), _I(vc), _I(0), _VP(o.data_ptr()), _LL(H * hd),
                              _VP(lse.data_ptr()), cu, _LL(total), _I(nseq), _I(max_t), _I(H), _I(KV), _I(hd),
                              _F(1.0 / math.sqrt(hd)), _VP(ops.status(q.device).data_ptr()), st)
    ops._rc(rc, "kb_flash_fwd")
    return o, lse


def flash_bwd(ops, do, q, k, v, o, lse, dq_out, dk_out, dv_out, which: int = 3) -> None:
    """Gradients written into the (strided) ``dq_out[B,T,H,hd]``, ``dk_out``/``dv_out[B,T,KV,hd]`` views."""
    B, T, H, hd = q.shape
    KV = k.shape[2]
    qs, qc = _rows(q)
    ks, kc = _rows(k)
    vs, vc = _rows(v)
    dos, doc = _rows(do)
    os_, _ = _rows(o)
    dqs, _ = _rows(dq_out)
    dks, _ = _rows(dk_out)
    dvs, _ = _rows(dv_out)
    dsum = torch.empty(B, H, T, device=q.device, dtype=torch.float32)
    st = _VP(torch.cuda.current_stream().cuda_stream)
    rc = ops.lib.kb_flash_bwd(_VP(q.data_ptr()), _LL(qs), _I(qc), _I(0), _VP(k.data_ptr()), _LL(ks), _I(kc), _I(0),
                              _VP(v.data_ptr()), _LL(vs), _I(vc), _I(0), _VP(o.data_ptr()), _LL(os_),
                              _VP(do.data_ptr()), _LL(dos), _I(doc), _I(0), _VP(lse.data_ptr()), _VP(dsum.data_ptr()),
                              _VP(dq_out.data_ptr()), _LL(dqs), _VP(dk_out.data_ptr()), _LL(dks),
                              _VP(dv_out.data_ptr()), _LL(dvs), _I(B), _I(T), _I(H), _I(KV), _I(hd),
                              _F(1.0 / math.sqrt(hd)), _I(which), _VP(ops.status(q.device).data_ptr()), st)
    ops._rc(rc, "kb_flash_bwd")
    ops.launches += 2          # D pre-pass, dK/dV and dQ kernels
