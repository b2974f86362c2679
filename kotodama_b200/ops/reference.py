"""Plain-PyTorch implementations of every fused op the training/serving executors use.

These define the numerics (statistics in fp32, outputs in the activation dtype) and are
the oracle for the sm_100a kernels in ``csrc/``; they are also the backend used on CPU
(fp32, gloo) runs.  Each function documents the tensor contract shared with its CUDA twin.

Math sources in the reference project: routing ``src/model/llama.py:630-644`` and its
Triton backward ``src/model/flash_attn_res/kernels/phase_1.py:204-249``; RMSNorm
``llama.py:143-153``; RoPE ``llama.py:172-203``; loss ``llama.py:837-849``.
"""
from __future__ import annotations

import contextlib

import math
from typing import Optional, Sequence

import torch
import torch.nn.functional as F


def _f(x: torch.Tensor) -> torch.Tensor:
    """Statistics dtype: fp32, or fp64 when the caller already works in fp64 (gradient checks)."""
    return x if x.dtype in (torch.float32, torch.float64) else x.float()


FP8_MAX = 448.0        # largest finite e4m3 value


class Fp8Weight:
    """A projection weight under the block-scaled fp8 recipe: the bf16 master (a view of the
    parameter arena) plus its e4m3 copies, 128x128-block scaled - ``q``/``s`` in the weight's own
    layout for the forward product, ``qt``/``st`` transposed for the data gradient.  ``refresh``
    re-quantises after the optimizer has changed the master.  Passing one of these where the GEMM
    ops expect the weight selects the fp8 path."""

    def __init__(self, w: torch.Tensor) -> None:
        self.w = w
        self.q = self.s = self.qt = self.st = None

    @property
    def shape(self):
        return self.w.shape

    def refresh(self, ops: "TorchOps") -> None:
        self.q, self.s, self.qt, self.st = ops.quant_blocks(self.w, transposed=True)


class DecodeWeight:
    """A projection weight of the serving engine: the K-major matrix ``w`` plus, on CUDA, a tile-major
    copy (``packed``: [N/128][K/64][128][64], 16 KB contiguous per tile) that the decode-size GEMM
    streams at DRAM page granularity.  Products with more than 128 rows (prefill) use ``w``."""

    def __init__(self, w: torch.Tensor, packed: Optional[torch.Tensor] = None) -> None:
        self.w, self.packed = w, packed

    @property
    def shape(self):
        return self.w.shape


def _to_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.clamp(-FP8_MAX, FP8_MAX).to(torch.float8_e4m3fn)


class TorchOps:
    """Backend object; ``CudaOps`` derives from it and overrides methods with kernels."""

    name = "torch"

    @contextlib.contextmanager
    def dependent_launch(self, on: bool = True):
        """Only the CUDA back end has launches to overlap."""
        yield

    def decode_weight(self, w: torch.Tensor) -> "DecodeWeight":
        """Wrap a serving projection weight; the CUDA backend adds the tile-major copy."""
        return DecodeWeight(w)

    # ------------------------------------------------------------------ block-scaled fp8
    fp8_pow2 = False      # scales rounded up to powers of two (what the hardware block-scaled GEMM takes)

    def _scale(self, amax: torch.Tensor) -> torch.Tensor:
        s = amax.clamp_min(1e-12) / FP8_MAX
        return torch.exp2(torch.ceil(torch.log2(s.double()))).float() if self.fp8_pow2 else s

    def quant_rows(self, x: torch.Tensor):
        """``x[M,K]`` -> e4m3 ``q[M,K]`` and scales ``s[K/128, M]`` (one per row and 128 columns)."""
        M, K = x.shape
        xb = x.float().view(M, K // 128, 128)
        s = self._scale(xb.abs().amax(-1))
        q = _to_e4m3(xb / s[..., None]).view(M, K)
        return q, s.t().contiguous()

    def quant_blocks(self, w: torch.Tensor, transposed: bool = False):
        """``w[N,K]`` -> e4m3 ``q[N,K]``, ``s[K/128, N/128]`` (128x128 blocks); with ``transposed``
        also ``qt[K,N]`` and ``st[N/128, K/128]``."""
        N, K = w.shape
        wb = w.float().view(N // 128, 128, K // 128, 128)
        s = self._scale(wb.abs().amax((1, 3)))                          # [N/128, K/128]
        q = _to_e4m3(wb / s[:, None, :, None]).view(N, K)
        if not transposed:
            return q, s.t().contiguous()
        return q, s.t().contiguous(), q.t().contiguous(), s.contiguous()

    def quant_cols_t(self, x: torch.Tensor):
        """``x[M,N]`` -> e4m3 ``qt[N,M]`` and scales ``s[M/128, N]`` (one per column and 128 rows)."""
        M, N = x.shape
        xb = x.float().view(M // 128, 128, N)
        s = self._scale(xb.abs().amax(1))                               # [M/128, N]
        q = _to_e4m3(xb / s[:, None, :]).view(M, N)
        return q.t().contiguous(), s.contiguous()

    def gemm_fp8(self, qa, sa, qb, sb, b_gran: int, out: Optional[torch.Tensor] = None, accumulate: bool = False,
                 out_dtype: torch.dtype = torch.bfloat16) -> torch.Tensor:
        """``sum_kb (qa_kb @ qb_kb^T) * sa[kb, m] * sb[kb, n // b_gran]`` with fp32 accumulation."""
        M, K = qa.shape
        N = qb.shape[0]
        a = qa.float().view(M, K // 128, 128) * sa.t()[..., None]
        sbe = sb if b_gran == 1 else sb.repeat_interleave(b_gran, dim=1)[:, :N]
        b = qb.float().view(N, K // 128, 128) * sbe.t()[..., None]
        r = a.view(M, K) @ b.view(N, K).t()
        if out is None:
            return r.to(out_dtype)
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r)
        return out

    def fp8_ok(self, *dims: int) -> bool:
        return all(d % 128 == 0 for d in dims)

    # ------------------------------------------------------------------ GEMM
    def gemm_nt(self, a: torch.Tensor, b, out: Optional[torch.Tensor] = None,
                residual: Optional[torch.Tensor] = None, accumulate: bool = False) -> torch.Tensor:
        """``a[M,K] @ b[N,K]^T (+ residual) -> [M,N]``; ``accumulate`` adds into ``out``.  ``b`` may be
        an ``Fp8Weight``: the product then runs in block-scaled fp8."""
        if isinstance(b, DecodeWeight):
            b = b.w
        if isinstance(b, Fp8Weight):
            if self.fp8_ok(a.shape[0], a.shape[1], b.shape[0]) and not accumulate:
                r = self.gemm_fp8(*self.quant_rows(a), b.q, b.s, 128, out_dtype=a.dtype)
                if residual is not None:
                    r = r + residual
                if out is not None:
                    out.copy_(r)
                    return out
                return r
            b = b.w
        r = a @ b.t()
        if residual is not None:
            r = r + residual
        if out is None:
            return r
        if accumulate:
            out.add_(r)
        else:
            out.copy_(r)
        return out

    def gemm_nn(self, a: torch.Tensor, b, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        """``a[M,K] @ b[K,N] -> [M,N]`` (data-gradient GEMM); ``b`` may be an ``Fp8Weight``."""
        if isinstance(b, Fp8Weight):
            if self.fp8_ok(a.shape[0], a.shape[1], b.shape[1]):
                return self.gemm_fp8(*self.quant_rows(a), b.qt, b.st, 128, out=out, out_dtype=a.dtype)
            b = b.w
        r = a @ b
        if out is None:
            return r
        out.copy_(r)
        return out

    def gemm_tn(self, a: torch.Tensor, b: torch.Tensor, out: Optional[torch.Tensor] = None,
                accumulate: bool = False, fp8: bool = False) -> torch.Tensor:
        """``a[K,M]^T @ b[K,N] -> [M,N]`` (weight-gradient GEMM, fp32 accumulation).  With ``fp8`` both
        operands are quantised in 128-token tiles and the product runs in block-scaled fp8."""
        if fp8 and self.fp8_ok(a.shape[0], a.shape[1], b.shape[1]):
            qa, sa = self.quant_cols_t(a)
            qb, sb = self.quant_cols_t(b)
            return self.gemm_fp8(qa, sa, qb, sb, 1, out=out, accumulate=accumulate, out_dtype=a.dtype)
        r = (a.t() @ b)
        if out is None:
            return r
        if accumulate:
            out.add_(r.to(out.dtype))
        else:
            out.copy_(r)
        return out

    # --------------------------------------------------- AttnRes route + norm
    def route_norm_fwd(self, srcs: Sequence[torch.Tensor], q: Optional[torch.Tensor],
                       rn_w: Optional[torch.Tensor], n_w: torch.Tensor, eps: float):
        """Fused depth-routing and RMSNorm.

        ``srcs``: S tensors ``[N,D]`` (committed blocks oldest first, then the partial).
        ``q``/``rn_w``: pseudo-query and key-norm weight ``[D]``; ``None`` means "no routing"
        (S must be 1, the source passes through).  ``n_w``: weight of the RMSNorm applied to the
        routed mixture.  Returns ``xn[N,D]`` and ``stats = (alpha[N,S], r[N,S], logit[N,S],
        rstd[N])`` in fp32.  The mixture itself is never materialised for the caller.
        """
        u = torch.stack([_f(s) for s in srcs], 1)              # [N,S,D]
        n, s, d = u.shape
        if q is None:
            assert s == 1
            alpha = torch.ones(n, 1, dtype=u.dtype, device=u.device)
            r = torch.zeros_like(alpha)
            logit = torch.zeros_like(alpha)
        else:
            w = _f((q * rn_w))
            r = torch.rsqrt(u.pow(2).mean(-1) + eps)
            logit = (u * w).sum(-1) * r
            alpha = torch.softmax(logit, 1)
        h = (alpha.unsqueeze(-1) * u).sum(1)
        rstd = torch.rsqrt(h.pow(2).mean(-1) + eps)
        xn = (h * rstd.unsqueeze(-1) * _f(n_w)).to(srcs[0].dtype)
        return xn, (alpha, r, logit, rstd)

    def route_norm_bwd(self, dxn: torch.Tensor, srcs: Sequence[torch.Tensor], q: Optional[torch.Tensor],
                       rn_w: Optional[torch.Tensor], n_w: torch.Tensor, eps: float, stats,
                       dsrcs: Sequence[torch.Tensor], acc: Sequence[bool]):
        """Backward of :meth:`route_norm_fwd`.

        Writes (``acc[s]`` False) or accumulates (True) the gradient of source ``s`` into
        ``dsrcs[s]`` and returns fp32 ``(dq, drn_w, dn_w)`` (the first two ``None`` without routing).
        """
        alpha, r, logit, rstd = stats
        u = torch.stack([_f(s) for s in srcs], 1)
        n, s, d = u.shape
        h = (alpha.unsqueeze(-1) * u).sum(1)
        hn = h * rstd.unsqueeze(-1)
        g = _f(dxn)
        dn_w = (g * hn).sum(0)
        gw = g * _f(n_w)
        dh = rstd.unsqueeze(-1) * (gw - hn * (gw * hn).mean(-1, keepdim=True))
        if q is None:
            du = dh.unsqueeze(1)
            dq = drn = None
        else:
            w = _f((q * rn_w))
            a = (dh.unsqueeze(1) * u).sum(-1)                           # [N,S]
            abar = (alpha * a).sum(1, keepdim=True)
            dl = alpha * (a - abar)
            du = alpha.unsqueeze(-1) * dh.unsqueeze(1) + dl.unsqueeze(-1) * (
                r.unsqueeze(-1) * w - (logit * r * r / d).unsqueeze(-1) * u)
            dw = ((dl * r).unsqueeze(-1) * u).sum((0, 1))
            dq, drn = dw * _f(rn_w), dw * _f(q)
        for j in range(s):
            if acc[j]:
                dsrcs[j].add_(du[:, j].to(dsrcs[j].dtype))
            else:
                dsrcs[j].copy_(du[:, j])
        return dq, drn, dn_w

    # --------------------------------------------------- AttnRes route, blocked form
    # One phase-1 pass over the committed sources serves every sub-layer query of a block; each
    # sub-layer then merges its own partial sum with a phase-2 step fused with the RMSNorm that
    # follows (reference: serve.py:113-164, kernels/phase_1.py:59-101, kernels/phase_2.py:9-57).
    def route_blocked_ok(self, S: int, D: int) -> bool:
        """Whether the blocked kernels cover ``S`` committed sources of width ``D`` (always, here)."""
        return True

    def route_p1_fwd(self, srcs: Sequence[torch.Tensor], qs: torch.Tensor, rn_ws: torch.Tensor, eps: float):
        """Phase 1 for ``Q`` queries at once.  ``srcs``: S committed sources ``[N,D]``; ``qs``/``rn_ws``
        ``[Q,D]`` pseudo-queries and key-norm weights.  Returns ``o[Q,N,D]`` (source dtype),
        ``lse[Q,N]`` fp32 and ``stats = (r[N,S], logit[Q,N,S])``."""
        u = torch.stack([_f(s) for s in srcs], 1)                       # [N,S,D]
        w = _f(qs) * _f(rn_ws)                                          # [Q,D]
        r = torch.rsqrt(u.pow(2).mean(-1) + eps)                        # [N,S]
        logit = torch.einsum("nsd,qd->qns", u, w) * r
        lse = torch.logsumexp(logit, -1)
        o = torch.einsum("qns,nsd->qnd", torch.softmax(logit, -1), u)
        return o.to(srcs[0].dtype), lse, (r, logit)

    def route_p2_fwd(self, o: torch.Tensor, lse: torch.Tensor, partial: Optional[torch.Tensor], q: torch.Tensor,
                     rn_w: torch.Tensor, n_w: torch.Tensor, eps: float):
        """Phase 2 + RMSNorm: merges the partial sum into one query's phase-1 result
        (``pi = sigmoid(l_p - lse)``, ``h = o + pi (p - o)``; ``partial`` None: ``h = o``) and normalises.
        Returns ``xn[N,D]`` and ``stats2[N,4]`` = (pi, l_p, r_p, rstd) fp32."""
        of = _f(o)
        n, d = of.shape
        if partial is None:
            pi = lp = rp = torch.zeros(n, dtype=of.dtype, device=of.device)
            h = of
        else:
            pf = _f(partial)
            w = _f(q) * _f(rn_w)
            rp = torch.rsqrt(pf.pow(2).mean(-1) + eps)
            lp = (pf * w).sum(-1) * rp
            pi = torch.sigmoid(lp - lse)
            h = of + pi.unsqueeze(-1) * (pf - of)
        rstd = torch.rsqrt(h.pow(2).mean(-1) + eps)
        xn = (h * rstd.unsqueeze(-1) * _f(n_w)).to(o.dtype)
        return xn, torch.stack([pi, lp, rp, rstd], 1)

    def route_p2_bwd(self, dxn: torch.Tensor, o: torch.Tensor, lse: torch.Tensor, partial: Optional[torch.Tensor],
                     q: torch.Tensor, rn_w: torch.Tensor, n_w: torch.Tensor, eps: float, stats2: torch.Tensor,
                     do_out: torch.Tensor, dlse_out: torch.Tensor, dpart: Optional[torch.Tensor], dpart_acc: bool):
        """Backward of :meth:`route_p2_fwd`: writes ``do_out[N,D]`` and ``dlse_out[N]``, writes or
        accumulates the partial's gradient into ``dpart`` and returns fp32 ``(dw, dn_w)`` where ``dw``
        is the gradient of ``q * rn_w`` (None without a partial)."""
        of, g = _f(o), _f(dxn)
        d = of.shape[1]
        pi, lp, rp, rstd = stats2.unbind(1)
        if partial is None:
            h = of
        else:
            pf = _f(partial)
            h = of + pi.unsqueeze(-1) * (pf - of)
        hn = h * rstd.unsqueeze(-1)
        dn_w = (g * hn).sum(0)
        gw = g * _f(n_w)
        dh = rstd.unsqueeze(-1) * (gw - hn * (gw * hn).mean(-1, keepdim=True))
        if partial is None:
            do_out.copy_(dh)
            dlse_out.zero_()
            return None, dn_w
        w = _f(q) * _f(rn_w)
        c = (dh * (of - pf)).sum(-1)
        dlse = pi * (1 - pi) * c
        dlp = -dlse
        dp = pi.unsqueeze(-1) * dh + dlp.unsqueeze(-1) * (rp.unsqueeze(-1) * w - (lp * rp * rp / d).unsqueeze(-1) * pf)
        dw = ((dlp * rp).unsqueeze(-1) * pf).sum(0)
        do_out.copy_((1 - pi).unsqueeze(-1) * dh)
        dlse_out.copy_(dlse)
        if dpart_acc:
            dpart.add_(dp.to(dpart.dtype))
        else:
            dpart.copy_(dp)
        return dw, dn_w

    def route_p1_bwd(self, srcs: Sequence[torch.Tensor], qs: torch.Tensor, rn_ws: torch.Tensor, do: torch.Tensor,
                     dlse: torch.Tensor, lse: torch.Tensor, stats, dsrcs: Sequence[torch.Tensor],
                     acc: Sequence[bool]) -> torch.Tensor:
        """Backward of :meth:`route_p1_fwd` for all ``Q`` queries at once: writes or accumulates the
        source gradients and returns ``dws[Q,D]`` fp32, the gradients of ``qs * rn_ws``
        (reference: kernels/phase_1.py:204-274)."""
        r, logit = stats
        u = torch.stack([_f(s) for s in srcs], 1)                       # [N,S,D]
        d = u.shape[-1]
        w = _f(qs) * _f(rn_ws)
        g = _f(do)                                                      # [Q,N,D]
        pr = torch.exp(logit - lse.unsqueeze(-1))                       # [Q,N,S]
        a = torch.einsum("qnd,nsd->qns", g, u)
        abar = (pr * a).sum(-1, keepdim=True)
        dl = pr * (dlse.unsqueeze(-1) + a - abar)
        du = (torch.einsum("qns,qnd->nsd", pr, g) + torch.einsum("qns,qd->nsd", dl * r, w)
              - ((dl * logit).sum(0) * r * r / d).unsqueeze(-1) * u)
        dws = torch.einsum("qns,nsd->qd", dl * r, u)
        for j in range(len(srcs)):
            if acc[j]:
                dsrcs[j].add_(du[:, j].to(dsrcs[j].dtype))
            else:
                dsrcs[j].copy_(du[:, j])
        return dws

    # ------------------------------------------------------ QK-norm + RoPE
    def qknorm_rope_fwd(self, qkv: torch.Tensor, qw: Optional[torch.Tensor], kw: Optional[torch.Tensor],
                        cos: torch.Tensor, sin: torch.Tensor, seq_len: int, n_q: int, n_kv: int, hd: int,
                        eps: float, pos_offset: int = 0, positions: Optional[torch.Tensor] = None, append=None):
        """Per-head RMSNorm (weight shared by heads) then rotate-half RoPE on the q and k parts of a
        fused ``qkv[N,(n_q+2*n_kv)*hd]`` projection.  Token ``n`` sits at position
        ``pos_offset + n % seq_len``.  Returns ``qk[N,(n_q+n_kv)*hd]`` and ``rstd[N,n_q+n_kv]`` (fp32)."""
        n = qkv.shape[0]
        nh = n_q + n_kv
        x = _f(qkv[:, : nh * hd].reshape(n, nh, hd))
        if qw is not None:
            rstd = torch.rsqrt(x.pow(2).mean(-1) + eps)
            w = torch.cat([_f(qw).expand(n_q, hd), _f(kw).expand(n_kv, hd)], 0)
            y = x * rstd.unsqueeze(-1) * w
        else:
            rstd = torch.ones(n, nh, dtype=x.dtype, device=qkv.device)
            y = x
        pos = (torch.arange(n, device=qkv.device) % seq_len) + pos_offset if positions is None else positions.long()
        c, s = _f(cos[pos]).unsqueeze(1), _f(sin[pos]).unsqueeze(1)
        h2 = hd // 2
        rot = torch.cat([-y[..., h2:], y[..., :h2]], -1)
        out = (y * c + rot * s).to(qkv.dtype).reshape(n, nh * hd)
        if append is not None:                           # serving: keys and values of the new tokens go to their cache slots
            k_pages, v_pages, slots = append
            self.kv_append(out[:, n_q * hd:], qkv[:, nh * hd:], k_pages, v_pages, slots)
        return out, rstd

    def qknorm_rope_bwd(self, dqk: torch.Tensor, qkv: torch.Tensor, qw, kw, cos, sin, rstd, seq_len: int,
                        n_q: int, n_kv: int, hd: int, dqkv_out: torch.Tensor, pos_offset: int = 0):
        """Backward: writes the q/k columns of ``dqkv_out[N,(n_q+2n_kv)*hd]`` and returns fp32
        ``(dqw, dkw)`` of shape ``[hd]`` (``None`` without QK-norm)."""
        n = qkv.shape[0]
        nh = n_q + n_kv
        pos = (torch.arange(n, device=qkv.device) % seq_len) + pos_offset
        c, s = _f(cos[pos]).unsqueeze(1), _f(sin[pos]).unsqueeze(1)
        g = _f(dqk.reshape(n, nh, hd))
        h2 = hd // 2
        gs = g * s
        dy = g * c + torch.cat([gs[..., h2:], -gs[..., :h2]], -1)   # transpose of the rotation
        if qw is None:
            dqkv_out[:, : nh * hd] = dy.reshape(n, nh * hd)
            return None, None
        x = _f(qkv[:, : nh * hd].reshape(n, nh, hd))
        xh = x * rstd.unsqueeze(-1)
        w = torch.cat([_f(qw).expand(n_q, hd), _f(kw).expand(n_kv, hd)], 0)
        dw_all = (dy * xh).sum(0)                                    # [nh,hd]
        dqw, dkw = dw_all[:n_q].sum(0), dw_all[n_q:].sum(0)
        gy = dy * w
        dx = rstd.unsqueeze(-1) * (gy - xh * (gy * xh).mean(-1, keepdim=True))
        dqkv_out[:, : nh * hd] = dx.reshape(n, nh * hd)
        return dqw, dkw

    # ------------------------------------------------------------ sampling
    @staticmethod
    def sample_uniform(seed: int, counter: int) -> float:
        """The sampler's random draw: splitmix64 of (seed, counter), top 24 bits, in [0, 1)."""
        m = (1 << 64) - 1
        z = (seed + 0x9E3779B97F4A7C15 * (counter + 1)) & m
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & m
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & m
        z ^= z >> 31
        return (z >> 40) / 16777216.0

    def sample(self, logits: torch.Tensor, temperature, top_k, top_p, rep_penalty, seeds, counters,
               seen: Optional[torch.Tensor], slots) -> torch.Tensor:
        """Next token per row of ``logits[B,V]`` in the reference's order (``serve.py:266-304``):
        repetition penalty (tokens whose bit is set in the request's ``seen`` bitmap row) ->
        temperature -> top-k (ties at the k-th value kept) -> top-p -> multinomial by inverse CDF in
        vocabulary order with ``u = sample_uniform(seed, counter)``; greedy at temperature 0.  The
        chosen token's bit is set in ``seen``.  Parameters are per-row sequences."""
        B, V = logits.shape
        out = torch.empty(B, dtype=torch.long)
        for b in range(B):
            v = logits[b].detach().float().cpu()
            row = seen[int(slots[b])] if seen is not None else None
            if row is not None and float(rep_penalty[b]) != 1.0:
                words = row.cpu().to(torch.int64) & 0xFFFFFFFF
                bits = ((words.unsqueeze(1) >> torch.arange(32)) & 1).flatten()[:V].bool()
                rp = float(rep_penalty[b])
                v = torch.where(bits, torch.where(v > 0, v / rp, v * rp), v)
            T = float(temperature[b])
            if T <= 0:
                tok = int(v.argmax())
            else:
                v = v / T
                k = int(top_k[b])
                keep = torch.ones(V, dtype=torch.bool)
                if 0 < k < V:
                    keep &= v >= torch.topk(v, k).values[-1]
                w = torch.where(keep, torch.exp(v - v.max()), torch.zeros_like(v))
                p = float(top_p[b])
                if 0.0 < p < 1.0:
                    srt, idx = torch.sort(torch.where(keep, v, torch.full_like(v, float("-inf"))), descending=True)
                    ws = w[idx]
                    before = ws.cumsum(0) - ws                     # mass of strictly earlier items
                    ok = (before <= p * float(w.sum())) & (ws > 0)
                    cut = srt[ok][-1] if bool(ok.any()) else srt[0]
                    w = torch.where(v >= cut, w, torch.zeros_like(w))    # ties at the threshold stay
                target = self.sample_uniform(int(seeds[b]), int(counters[b])) * float(w.sum())
                cdf = w.cumsum(0)
                hit = ((cdf > target) & (w > 0)).nonzero()
                tok = int(hit[0]) if hit.numel() else int((w > 0).nonzero()[-1])
            out[b] = tok
            if row is not None:
                word = int(row[tok >> 5].item()) & 0xFFFFFFFF
                word |= 1 << (tok & 31)
                row[tok >> 5] = word - (1 << 32) if word >= (1 << 31) else word
        return out.to(logits.device)

    # ------------------------------------------------------------ attention
    def attention_fwd(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, need_grad: bool = True,
                      cu_seqlens: Optional[torch.Tensor] = None, max_seqlen: int = 0):
        """Causal GQA attention.  ``q[B,T,H,hd]``, ``k,v[B,T,KV,hd]`` (may be strided views);
        returns ``o[B,T,H,hd]`` contiguous and ``lse[B,H,T]`` fp32 (natural log).  With ``cu_seqlens``
        the single batch row holds several sequences back to back (``lse`` is then ``[H, total]``)."""
        if cu_seqlens is not None:
            cu = cu_seqlens.tolist()
            outs = [self.attention_fwd(q[:, a:e], k[:, a:e], v[:, a:e], need_grad) for a, e in zip(cu[:-1], cu[1:])]
            return torch.cat([o for o, _ in outs], 1), torch.cat([l[0] for _, l in outs], 1)
        b, t, h, hd = q.shape
        kv = k.shape[2]
        g = h // kv
        qf = _f(q).permute(0, 2, 1, 3)
        kf = _f(k).permute(0, 2, 1, 3).repeat_interleave(g, 1)
        vf = _f(v).permute(0, 2, 1, 3).repeat_interleave(g, 1)
        sc = (qf @ kf.transpose(-1, -2)) / math.sqrt(hd)
        mask = torch.ones(t, t, dtype=torch.bool, device=q.device).tril()
        sc = sc.masked_fill(~mask, float("-inf"))
        lse = torch.logsumexp(sc, -1)
        o = torch.softmax(sc, -1) @ vf
        return o.permute(0, 2, 1, 3).contiguous().to(q.dtype), lse

    def attention_bwd(self, do, q, k, v, o, lse, dq_out, dk_out, dv_out) -> None:
        """Gradients of :meth:`attention_fwd` written into the (possibly strided) ``d*_out`` views."""
        b, t, h, hd = q.shape
        kv = k.shape[2]
        g = h // kv
        qf = _f(q).permute(0, 2, 1, 3)
        kf = _f(k).permute(0, 2, 1, 3).repeat_interleave(g, 1)
        vf = _f(v).permute(0, 2, 1, 3).repeat_interleave(g, 1)
        dof = _f(do).permute(0, 2, 1, 3)
        of = _f(o).permute(0, 2, 1, 3)
        scale = 1.0 / math.sqrt(hd)
        sc = (qf @ kf.transpose(-1, -2)) * scale
        mask = torch.ones(t, t, dtype=torch.bool, device=q.device).tril()
        p = torch.exp(sc - lse.unsqueeze(-1)).masked_fill(~mask, 0.0)
        dv = p.transpose(-1, -2) @ dof
        dp = dof @ vf.transpose(-1, -2)
        delta = (dof * of).sum(-1, keepdim=True)
        ds = p * (dp - delta) * scale
        dq = ds @ kf
        dk = ds.transpose(-1, -2) @ qf
        dq_out.copy_(dq.permute(0, 2, 1, 3))
        dk_out.copy_(dk.view(b, kv, g, t, hd).sum(2).permute(0, 2, 1, 3))
        dv_out.copy_(dv.view(b, kv, g, t, hd).sum(2).permute(0, 2, 1, 3))

    # -------------------------------------------------------------- SwiGLU
    def swiglu_fwd(self, gu: torch.Tensor) -> torch.Tensor:
        """``silu(gate) * up`` for ``gu = [gate | up]`` of shape ``[N,2F]``."""
        f = gu.shape[1] // 2
        g, u = _f(gu[:, :f]), _f(gu[:, f:])
        return (F.silu(g) * u).to(gu.dtype)

    def swiglu_bwd(self, gu: torch.Tensor, dact: torch.Tensor, out: Optional[torch.Tensor] = None) -> torch.Tensor:
        f = gu.shape[1] // 2
        g, u, d = _f(gu[:, :f]), _f(gu[:, f:]), _f(dact)
        sg = torch.sigmoid(g)
        dg = d * u * sg * (1 + g * (1 - sg))
        du = d * g * sg
        r = torch.cat([dg, du], 1).to(gu.dtype)
        if out is None:
            return r
        out.copy_(r)
        return out

    # ------------------------------------------------- LM head + CE + z-loss
    def linear_ce(self, h: torch.Tensor, w: torch.Tensor, labels: torch.Tensor, z_weight: float,
                  grad_scale: float, dw: Optional[torch.Tensor], dw_accumulate: bool, chunk: int = 4096,
                  need_grad: bool = True, count: Optional[torch.Tensor] = None):
        """Chunked LM-head GEMM + cross-entropy + z-loss without materialising all logits.

        ``labels[N]`` uses -100 for ignored rows.  Losses are means over the valid rows:
        returns ``(ce_mean, z_mean_weighted, dh)`` where ``dh`` (and ``dw``, accumulated into the
        given buffer) are gradients of ``grad_scale * (ce + z)``.
        """
        n = h.shape[0]
        valid = labels >= 0
        nv = valid.sum().clamp(min=1).to(torch.float64 if h.dtype == torch.float64 else torch.float32)
        if count is not None:          # the batch is split over ranks: normalise by the global count
            nv = count.reshape(()).to(nv.dtype)
        acc_dt = torch.float64 if h.dtype == torch.float64 else torch.float32
        ce_sum = torch.zeros((), dtype=acc_dt, device=h.device)
        z_sum = torch.zeros((), dtype=acc_dt, device=h.device)
        dh = torch.empty_like(h) if need_grad else None
        first = not dw_accumulate
        for s in range(0, n, chunk):
            hc, lc, vc = h[s:s + chunk], labels[s:s + chunk], valid[s:s + chunk]
            logits = _f(self.gemm_nt(hc, w))
            lse = torch.logsumexp(logits, -1)
            tgt = logits.gather(1, lc.clamp(min=0).unsqueeze(1)).squeeze(1)
            ce_sum += ((lse - tgt) * vc).sum()
            z_sum += ((lse * lse) * vc).sum()
            if need_grad:
                p = torch.softmax(logits, -1)
                dl = p * (1.0 + 2.0 * z_weight * lse).unsqueeze(1)
                dl.scatter_add_(1, lc.clamp(min=0).unsqueeze(1), -torch.ones_like(lse).unsqueeze(1))
                dl = (dl * (vc.to(nv.dtype) * grad_scale / nv).unsqueeze(1)).to(h.dtype)
                self.gemm_nn(dl, w, out=dh[s:s + chunk])
                if dw is not None:
                    self.gemm_tn(dl, hc, out=dw, accumulate=not first)
                    first = False
        return ce_sum / nv, z_weight * z_sum / nv, dh

    # ----------------------------------------------------------- embedding
    def embedding_fwd(self, ids: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        return w[ids]

    def embedding_bwd(self, dout: torch.Tensor, ids: torch.Tensor, dw: torch.Tensor) -> None:
        """``dw[ids[n]] += dout[n]`` (duplicates sum)."""
        dw.index_add_(0, ids, dout.to(dw.dtype))

    # ------------------------------------------------------- optimizer math
    def sumsq(self, x: torch.Tensor) -> torch.Tensor:
        return _f(x).pow(2).sum()

    def adamw_step(self, p: torch.Tensor, g: torch.Tensor, m: torch.Tensor, v: torch.Tensor, step: int,
                   lr: float, b1: float, b2: float, eps: float, wd: float, gscale) -> None:
        """Decoupled AdamW on flat tensors; ``gscale`` (float or 0-dim tensor) multiplies the gradient."""
        gf = _f(g) * gscale
        m.mul_(b1).add_(gf.to(m.dtype), alpha=1 - b1)
        v.mul_(b2).add_((gf * gf).to(v.dtype), alpha=1 - b2)
        bc1, bc2 = 1 - b1 ** step, 1 - b2 ** step
        pf = _f(p) * (1 - lr * wd)
        pf = pf - (lr / bc1) * _f(m) / (_f(v).sqrt() / math.sqrt(bc2) + eps)
        p.copy_(pf)

    def muon_momentum(self, g: torch.Tensor, buf: torch.Tensor, momentum: float, nesterov: bool, gscale):
        """``buf = m*buf + g*gscale``; returns the Nesterov update ``m*buf + g*gscale`` in fp16 together with
        its squared Frobenius norm (fp32, 0-dim)."""
        gf = (_f(g) * gscale).to(g.dtype)
        buf.mul_(momentum).add_(gf)
        upd = (momentum * buf + gf) if nesterov else buf.clone()
        x = upd.half()
        return x, _f(x).pow(2).sum()

    def ns_normalize(self, x: torch.Tensor, sumsq: torch.Tensor) -> torch.Tensor:
        """``x / (||x||_F + 1e-7)`` with the squared norm supplied (``muon.py:142``)."""
        return (_f(x) / (sumsq.sqrt() + 1e-7)).to(x.dtype)

    def ns_iteration(self, x: torch.Tensor, a: float, b: float, c: float) -> torch.Tensor:
        """One Newton-Schulz step on ``x[R,C]`` (R<=C) or a batch ``x[n,R,C]`` of same-shape matrices,
        fp16 operands (``muon.py:144-147``, batching as in ``muon.py:155-188``)."""
        A = x @ x.transpose(-1, -2)
        B = b * A + c * (A @ A)
        return a * x + B @ x

    def muon_apply(self, p: torch.Tensor, orth: torch.Tensor, lr: float, wd: float, scale: float,
                   transposed: bool) -> None:
        """``p = p*(1-lr*wd) - lr*scale*orth`` (orth given transposed when the matrix was tall)."""
        o = orth.t() if transposed else orth
        if wd > 0:
            p.mul_(1 - lr * wd)
        p.add_(o.to(p.dtype), alpha=-lr * scale)

    def transpose(self, x: torch.Tensor) -> torch.Tensor:
        return x.t().contiguous()


    # ------------------------------------------------------------- serving
    def kv_append(self, k, v, k_pages, v_pages, slots) -> None:
        """Copy rows ``k[n], v[n]`` (``[N, n_kv*hd]``) into cache slot ``slots[n]`` (= page*16 + offset)."""
        n_kv, hd = k_pages.shape[1], k_pages.shape[3]          # cache layout [pages, n_kv, 16, hd]
        ok = slots >= 0
        s = slots[ok]
        k_pages[s // 16, :, s % 16] = k[ok].reshape(-1, n_kv, hd)
        v_pages[s // 16, :, s % 16] = v[ok].reshape(-1, n_kv, hd)

    def paged_decode_attention(self, q, k_pages, v_pages, page_table, ctx_lens, max_ctx, n_q, n_kv, hd, split=512):
        """One query token per request against its pages (``k_pages[P,n_kv,16,hd]``)."""
        B = q.shape[0]
        g = n_q // n_kv
        out = torch.empty(B, n_q * hd, device=q.device, dtype=q.dtype)
        for b in range(B):
            n = int(ctx_lens[b])
            pages = page_table[b, : (n + 15) // 16].long()
            k = _f(k_pages[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, hd)[:, :n]).repeat_interleave(g, 0)
            v = _f(v_pages[pages].permute(1, 0, 2, 3).reshape(n_kv, -1, hd)[:, :n]).repeat_interleave(g, 0)
            qb = _f(q[b]).view(n_q, 1, hd)
            p = torch.softmax((qb @ k.transpose(1, 2)) / math.sqrt(hd), -1)
            out[b] = (p @ v).reshape(-1).to(q.dtype)
        return out

    def argmax(self, logits: torch.Tensor) -> torch.Tensor:
        return logits.float().argmax(-1)


TORCH_OPS = TorchOps()
