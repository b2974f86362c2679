"""sm_100a backend: the same op contract as :class:`TorchOps`, carried out by the kernels in
``csrc/`` through ``ctypes`` (raw pointers + the current CUDA stream).

Activations and parameters are bf16, statistics fp32, Newton-Schulz operands fp16.  A GEMM
whose operands break the TMA rules (16-byte aligned base, leading dimension a multiple of 8
elements) raises instead of taking another path.  Kernels that wait (mbarrier pipelines) bound
their waits and report through a device status word, read by :meth:`CudaOps.check_status`.
"""
from __future__ import annotations

import contextlib
import ctypes
import math
from typing import Optional, Sequence

import torch

from . import _build
from .reference import DecodeWeight, Fp8Weight, TorchOps

_VP = ctypes.c_void_p
_I = ctypes.c_int
_LL = ctypes.c_longlong
_F = ctypes.c_float

_FMT = {torch.float16: 0, torch.bfloat16: 1}
_OUT = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _p(t: Optional[torch.Tensor]) -> _VP:
    return _VP(t.data_ptr()) if t is not None else _VP(None)


def _st() -> _VP:
    return _VP(torch.cuda.current_stream().cuda_stream)


class KernelError(RuntimeError):
    pass


class CudaOps(TorchOps):
    name = "sm100"

    def __init__(self, gemm_backend: str = "tcgen05", attention_backend: str = "auto") -> None:
        self.lib = _build.load()
        import os
        self.gemm_backend = os.environ.get("KOTODAMA_GEMM", gemm_backend)   # "cublas" = library baseline
        self.attention_backend = attention_backend
        self.mn_major = os.environ.get("KOTODAMA_MN_MAJOR", "1") == "1"   # MN-major GEMM operands (no transposes)
        self.launches = 0              # launches of kernels from this library
        self._status: dict[int, torch.Tensor] = {}
        self.gemm_max_ctas = 0
        self.split_k_small_m = True
        self._splitk_ws: dict = {}
        self.attention_library_calls = 0   # stays 0: attention runs on the native kernels in both directions
        self.gemm_2cta = os.environ.get("KOTODAMA_GEMM_2CTA", "1") == "1"   # CTA-pair kernel for large products
        # fp8 products: "mx" = hardware block-scaled MMA (power-of-two scales, accumulation stays in tensor
        # memory); "promote" = fp32 scales applied per K block in registers
        self.skinny_cluster = os.environ.get("KOTODAMA_SKINNY", "cluster") != "splitk"   # decode-size GEMMs: cluster split-K through DSMEM
        self._merge_counters: dict = {}
        # split merge of the decode attention: its own (dependent) launch, or inside the decode kernel by the last CTA
        # of a (request, kv head) pair.  Measured on the 3B decode step: 4.18 ms with the launch, 4.37 ms fused (the
        # device-wide fence and the election at the end of 2560 CTAs cost more than 28 short launches), so: launch
        self.decode_merge_fused = os.environ.get("KOTODAMA_DECODE_MERGE", "kernel") == "fused"
        self.pack_decode_weights = os.environ.get("KOTODAMA_PACK_DECODE", "0") == "1"   # serving: tile-major weight copies for decode (measured +3 %, costs a second copy of the weights: off)
        self.fp8_backend = os.environ.get("KOTODAMA_FP8", "mx")
        self.fp8_pow2 = self.fp8_backend == "mx"
        self.fp8_pair = int(os.environ.get("KOTODAMA_FP8_PAIR", "0"))       # mx kernel: 1 = SM-pair tiles, 0 = one CTA per tile (faster, default)
        for name in ("kb_route_bwd_grid", "kb_qknorm_grid_warps", "kb_route_pipe_grid", "kb_route_blocked_ok",
                     "kb_route_blocked_grid"):
            getattr(self.lib, name).restype = _I

    # ------------------------------------------------------------------ utils
    def _rc(self, rc: int, what: str) -> None:
        self.launches += 1
        if rc != 0:
            raise KernelError(f"{what}: launcher returned {rc}")

    def _call(self, fn: str, *args) -> None:
        self._rc(getattr(self.lib, fn)(*args), fn)

    def status(self, device: torch.device) -> torch.Tensor:
        idx = device.index if device.index is not None else torch.cuda.current_device()
        if idx not in self._status:
            self._status[idx] = torch.zeros(1, dtype=torch.int32, device=device)
        return self._status[idx]

    def check_status(self, device: Optional[torch.device] = None) -> None:
        """Host-side check of the bounded-wait status word (synchronises)."""
        for idx, t in self._status.items():
            v = int(t.item())
            if v != 0:
                t.zero_()
                what = {5: "a kernel refused its arguments", 6: "an index read from data (token id, label or cache slot) "
                        "was out of range; the access was skipped"}.get(v, "a kernel wait timed out")
                raise KernelError(f"device {idx}: {what} (status {v})")
        if self._status:        # the decode kernels keep their own status word (no status argument)
            torch.cuda.synchronize()
            v = int(self.lib.kb_decode_status())
            if v != 0:
                raise KernelError(f"paged decode attention: a bulk copy did not arrive in time (status {v})")

    # ------------------------------------------------------------------ GEMM
    def _gemm(self, a: torch.Tensor, b: torch.Tensor, M: int, N: int, K: int, a_mn: bool, b_mn: bool,
              out: Optional[torch.Tensor] = None, cin: Optional[torch.Tensor] = None, alpha: float = 1.0,
              beta: float = 0.0, out_dtype: Optional[torch.dtype] = None, batch: int = 1,
              sym_upper: bool = False, diag: float = 0.0, b_const: bool = False) -> torch.Tensor:
        """``b_const``: ``b`` is a weight that nothing writes while kernels are in flight (serving), so a
        decode-size product launched as a dependent may fetch it before the kernels ahead have finished.
        ``diag`` is added to the diagonal of the result (fused into the CTA-pair kernel's epilogue when
        there is an addend, a separate in-place add otherwise)."""
        out_dtype = out_dtype or (out.dtype if out is not None else a.dtype)
        lead = (batch,) if batch > 1 else ()
        if out is None:
            out = torch.empty(*lead, M, N, device=a.device, dtype=out_dtype)
        if self.gemm_backend == "cublas":
            # library arm for A/B runs: one cuBLAS call with alpha/beta where the dtypes allow it (no
            # fp32 round trip, no extra passes over the result), so that the comparison is fair
            am = a.transpose(-1, -2) if a_mn else a
            bm = b if b_mn else b.transpose(-1, -2)
            same = out.dtype == a.dtype == b.dtype and (cin is None or cin.dtype == out.dtype)
            if same and cin is None and alpha == 1.0:
                torch.matmul(am, bm, out=out)
            elif same and batch == 1:
                torch.addmm(cin if cin is not None else out, am, bm, beta=beta if cin is not None else 0.0, alpha=alpha, out=out)
            elif same:
                torch.baddbmm(cin if cin is not None else out, am, bm, beta=beta if cin is not None else 0.0, alpha=alpha, out=out)
            else:                                  # mixed dtypes (fp32 accumulation targets): library product, then one fused pass
                r = torch.matmul(am, bm)
                if cin is not None:
                    torch.add(cin.to(out.dtype) * beta, r.to(out.dtype), alpha=alpha, out=out)
                else:
                    out.copy_(r if alpha == 1.0 else r * alpha)
            if diag:
                out.diagonal(dim1=-2, dim2=-1).add_(diag)
            return out
        for t in (a, b):
            if t.stride(-1) != 1 or t.stride(-2) % 8 or t.data_ptr() % 16 or t.dtype not in _FMT:
                raise KernelError(f"GEMM operand not TMA-compatible: shape {tuple(t.shape)} stride {t.stride()} {t.dtype}")
        if out.stride(-1) != 1 or (cin is not None and (cin.stride(-1) != 1 or cin.dtype != out.dtype)):
            raise KernelError("GEMM output/addend must be row-major and of one dtype")
        bs = lambda t: t.stride(0) if batch > 1 else 0
        tiles = ((M + 127) // 128) * ((N + 255) // 256)
        kblocks = (K + 63) // 64
        if (batch == 1 and M <= 128 and tiles <= 74 and kblocks >= 8 and out.dtype == torch.bfloat16
                and out.is_contiguous() and (cin is None or cin.is_contiguous()) and self.split_k_small_m):
            # skinny (decode-size) products: too few output tiles to fill the GPU.  bf16 K-major operands: the K
            # range is split over the CTAs of a thread-block cluster and the partial tiles are summed through
            # distributed shared memory (one launch); otherwise split-K with fp32 atomics and a finishing kernel
            if (self.skinny_cluster and not a_mn and not b_mn and a.dtype == torch.bfloat16 and b.dtype == torch.bfloat16
                    and not diag):
                rc = self.lib.kb_gemm_skinny(_p(a), _p(b), _p(out), _p(cin), _I(M), _I(N), _I(K), _LL(a.stride(-2)),
                                             _LL(b.stride(-2)), _LL(out.stride(-2)),
                                             _LL(cin.stride(-2) if cin is not None else 0), _F(alpha), _F(beta), _I(0),
                                             _I(0), _I(2 if b_const else 0), _p(self.status(a.device)), _st())
                if rc == 0:
                    self.launches += 1
                    return out
                if rc != 9:                          # 9: the runtime could not place the cluster - use the atomics path
                    self._rc(rc, "kb_gemm_skinny")
                self.skinny_cluster = False
            split = max(2, min(148 // tiles, kblocks // 2, 16))
            # one fp32 workspace per output size, zeroed once: the finishing kernel clears it again
            key = (M * N, a.device.index)
            ws = self._splitk_ws.get(key)
            if ws is None:
                ws = self._splitk_ws[key] = torch.zeros(M * N, device=a.device, dtype=torch.float32)
            rc = self.lib.kb_gemm(_p(a), _p(b), _p(ws), _p(None), _I(M), _I(N), _I(K), _I(1),
                                  _LL(a.stride(-2)), _LL(b.stride(-2)), _LL(N), _LL(0), _LL(0), _LL(0), _LL(0), _LL(0),
                                  _I(int(a_mn)), _I(int(b_mn)), _I(_FMT[a.dtype]), _I(_FMT[b.dtype]), _I(2),
                                  _F(alpha), _F(0.0), _p(self.status(a.device)), _I(self.gemm_max_ctas), _I(split),
                                  _st())
            self._rc(rc, "kb_gemm(split-k)")
            self._rc(self.lib.kb_f32_to_bf16_add(_p(ws), _p(cin), _F(beta), _p(out), _LL(M * N), _I(1), _st()),
                     "kb_f32_to_bf16_add")
            if diag:
                out.diagonal(dim1=-2, dim2=-1).add_(diag)
            return out
        if self.gemm_2cta and M >= 256 and N >= 256:
            # large products: CTA pairs (256x256 tiles, tcgen05 cta_group::2)
            rc = self.lib.kb_gemm_2cta(_p(a), _p(b), _p(out), _p(cin), _I(M), _I(N), _I(K), _I(batch),
                                       _LL(a.stride(-2)), _LL(b.stride(-2)), _LL(out.stride(-2)),
                                       _LL(cin.stride(-2) if cin is not None else 0),
                                       _LL(bs(a)), _LL(bs(b)), _LL(bs(out)), _LL(bs(cin) if cin is not None else 0),
                                       _I(int(a_mn)), _I(int(b_mn)), _I(_FMT[a.dtype]), _I(_FMT[b.dtype]),
                                       _I(_OUT[out.dtype]), _F(alpha), _F(beta), _p(self.status(a.device)),
                                       _I(self.gemm_max_ctas), _I(int(sym_upper)), _F(diag if cin is not None else 0.0), _st())
            self._rc(rc, "kb_gemm_2cta")
            if diag and cin is None:
                out.diagonal(dim1=-2, dim2=-1).add_(diag)
            # sym_upper: only tiles on/above the diagonal are computed; the epilogue writes each of them
            # to its mirrored position as well (16-bit outputs)
            if sym_upper and out.dtype == torch.float32:
                self._rc(self.lib.kb_mirror_upper16(_p(out), _I(M), _LL(out.stride(-2)), _I(batch), _LL(bs(out)),
                                                    _st()), "kb_mirror_upper16")
            return out
        rc = self.lib.kb_gemm(_p(a), _p(b), _p(out), _p(cin), _I(M), _I(N), _I(K), _I(batch),
                              _LL(a.stride(-2)), _LL(b.stride(-2)), _LL(out.stride(-2)),
                              _LL(cin.stride(-2) if cin is not None else 0),
                              _LL(bs(a)), _LL(bs(b)), _LL(bs(out)), _LL(bs(cin) if cin is not None else 0),
                              _I(int(a_mn)), _I(int(b_mn)), _I(_FMT[a.dtype]), _I(_FMT[b.dtype]), _I(_OUT[out.dtype]),
                              _F(alpha), _F(beta), _p(self.status(a.device)), _I(self.gemm_max_ctas), _I(1), _st())
        self._rc(rc, "kb_gemm")
        if diag:
            out.diagonal(dim1=-2, dim2=-1).add_(diag)
        return out

    # ------------------------------------------------------------------ block-scaled fp8
    def quant_rows(self, x):
        M, K = x.shape
        x = x.contiguous()
        q = torch.empty(M, K, device=x.device, dtype=torch.float8_e4m3fn)
        s = torch.empty(K // 128, M, device=x.device, dtype=torch.float32)
        self._call("kb_quant_rows", _p(x), _LL(K), _p(q), _LL(K), _p(s), _I(M), _I(K), _I(int(self.fp8_pow2)), _st())
        return q, s

    def quant_blocks(self, w, transposed=False):
        N, K = w.shape
        w = w.contiguous()
        dev = w.device
        q = torch.empty(N, K, device=dev, dtype=torch.float8_e4m3fn)
        s = torch.empty(K // 128, N // 128, device=dev, dtype=torch.float32)
        qt = torch.empty(K, N, device=dev, dtype=torch.float8_e4m3fn) if transposed else None
        st = torch.empty(N // 128, K // 128, device=dev, dtype=torch.float32) if transposed else None
        self._call("kb_quant_blocks", _p(w), _LL(K), _p(q), _p(s), _p(qt), _p(st), _I(N), _I(K), _I(int(self.fp8_pow2)), _st())
        return (q, s, qt, st) if transposed else (q, s)

    def quant_cols_t(self, x):
        M, N = x.shape
        x = x.contiguous()
        qt = torch.empty(N, M, device=x.device, dtype=torch.float8_e4m3fn)
        s = torch.empty(M // 128, N, device=x.device, dtype=torch.float32)
        self._call("kb_quant_cols_t", _p(x), _LL(N), _p(qt), _p(s), _I(M), _I(N), _I(int(self.fp8_pow2)), _st())
        return qt, s

    def gemm_fp8(self, qa, sa, qb, sb, b_gran, out=None, accumulate=False, out_dtype=torch.bfloat16, residual=None):
        M, K = qa.shape
        N = qb.shape[0]
        if out is None:
            out = torch.empty(M, N, device=qa.device, dtype=out_dtype)
        cin = residual if residual is not None else (out if accumulate else None)
        otype = {torch.bfloat16: 1, torch.float32: 2}[out.dtype]
        self._call("kb_gemm_mxfp8" if self.fp8_backend == "mx" else "kb_gemm_fp8", _p(qa), _p(qb), _p(sa), _p(sb), _p(out), _p(cin), _I(M), _I(N), _I(K), _LL(K), _LL(K),
                   _LL(out.stride(0)), _I(b_gran), _I(sb.shape[1]), _I(otype), _F(1.0), _F(1.0 if cin is not None else 0.0),
                   _p(self.status(qa.device)), _I(self.fp8_pair if self.fp8_backend == "mx" else 0), _st())
        return out

    @contextlib.contextmanager
    def dependent_launch(self, on: bool = True):
        """Inside the block the decode-path kernels (routing + norm forward, QK-norm + RoPE, cache append, decode
        attention and its merge, SwiGLU, the decode-size product) are launched as programmatic dependents of
        the kernel before them: their launch and prologue - for the product also the first ring-full of weight
        tiles - overlap that kernel's tail.  A CUDA graph captured inside the block keeps the edges."""
        was = self.lib.kb_set_dependent_launch(_I(1 if on else 0))
        try:
            yield
        finally:
            self.lib.kb_set_dependent_launch(_I(was))

    def decode_weight(self, w: torch.Tensor) -> DecodeWeight:
        N, K = w.shape
        if not (self.skinny_cluster and self.pack_decode_weights and w.is_cuda and w.dtype == torch.bfloat16
                and w.is_contiguous() and K % 64 == 0):
            return DecodeWeight(w)
        packed = torch.empty(((N + 127) // 128) * (K // 64) * 8192, device=w.device, dtype=torch.bfloat16)
        self._call("kb_pack_weight_tiles", _p(w), _LL(K), _p(packed), _I(N), _I(K), _st())
        return DecodeWeight(w, packed)

    def gemm_nt(self, a, b, out=None, residual=None, accumulate=False):
        b_const = isinstance(b, DecodeWeight)
        if b_const:
            M, K = a.shape
            N = b.w.shape[0]
            if (b.packed is not None and self.skinny_cluster and M <= 128 and a.dtype == torch.bfloat16
                    and a.stride(-1) == 1 and a.stride(-2) % 8 == 0 and a.data_ptr() % 16 == 0
                    and (N + 255) // 256 <= 74 and K >= 512):
                if out is None:
                    out = torch.empty(M, N, device=a.device, dtype=torch.bfloat16)
                cin = residual if residual is not None else (out if accumulate else None)
                if out.stride(-1) == 1 and (cin is None or (cin.stride(-1) == 1 and cin.dtype == out.dtype)):
                    rc = self.lib.kb_gemm_skinny(_p(a), _p(b.packed), _p(out), _p(cin), _I(M), _I(N), _I(K), _LL(a.stride(-2)),
                                                 _LL(K), _LL(out.stride(-2)), _LL(cin.stride(-2) if cin is not None else 0),
                                                 _F(1.0), _F(1.0), _I(0), _I(0), _I(3), _p(self.status(a.device)), _st())
                    if rc == 0:
                        self.launches += 1
                        return out
                    if rc != 9:
                        self._rc(rc, "kb_gemm_skinny(packed)")
                    self.skinny_cluster = False
            b = b.w
        if isinstance(b, Fp8Weight):
            if self.fp8_ok(a.shape[0], a.shape[1], b.shape[0]) and a.dtype == torch.bfloat16 and not (
                    accumulate and residual is not None):
                qa, sa = self.quant_rows(a)
                return self.gemm_fp8(qa, sa, b.q, b.s, 128, out=out, accumulate=accumulate, residual=residual)
            b = b.w
        cin = residual if residual is not None else (out if accumulate else None)
        return self._gemm(a, b, a.shape[0], b.shape[0], a.shape[1], False, False, out, cin, 1.0, 1.0, b_const=b_const)

    def gemm_nn(self, a, b, out=None):
        if isinstance(b, Fp8Weight):
            if self.fp8_ok(a.shape[0], a.shape[1], b.shape[1]) and a.dtype == torch.bfloat16:
                qa, sa = self.quant_rows(a)
                return self.gemm_fp8(qa, sa, b.qt, b.st, 128, out=out)
            b = b.w
        if self.mn_major:
            return self._gemm(a, b, a.shape[0], b.shape[1], a.shape[1], False, True, out)
        return self._gemm(a, self.transpose(b), a.shape[0], b.shape[1], a.shape[1], False, False, out)

    def gemm_tn(self, a, b, out=None, accumulate=False, fp8=False):
        if fp8 and self.fp8_ok(a.shape[0], a.shape[1], b.shape[1]) and a.dtype == torch.bfloat16:
            qa, sa = self.quant_cols_t(a)
            qb, sb = self.quant_cols_t(b)
            return self.gemm_fp8(qa, sa, qb, sb, 1, out=out, accumulate=accumulate)
        cin = out if accumulate else None
        if self.mn_major:
            return self._gemm(a, b, a.shape[1], b.shape[1], a.shape[0], True, True, out, cin, 1.0, 1.0)
        return self._gemm(self.transpose(a), self.transpose(b), a.shape[1], b.shape[1], a.shape[0], False, False,
                          out, cin, 1.0, 1.0)

    # ------------------------------------------------------------------ routing
    def route_norm_fwd(self, srcs: Sequence[torch.Tensor], q, rn_w, n_w, eps: float):
        S = len(srcs)
        N, D = srcs[0].shape
        dev = srcs[0].device
        xn = torch.empty(N, D, device=dev, dtype=torch.bfloat16)
        routing = q is not None
        alpha = torch.empty(N, S, device=dev, dtype=torch.float32) if routing else None
        r = torch.empty(N, S, device=dev, dtype=torch.float32) if routing else None
        logit = torch.empty(N, S, device=dev, dtype=torch.float32) if routing else None
        rstd = torch.empty(N, device=dev, dtype=torch.float32)
        arr = (_VP * S)(*[s.data_ptr() for s in srcs])
        if self.lib.kb_route_pipe_grid(_I(N), _I(S), _I(D), _I(0)) > 0:
            rc = self.lib.kb_route_pipe_fwd(arr, _I(S), _p(q), _p(rn_w), _p(n_w), _p(xn), _p(alpha), _p(r), _p(logit),
                                            _p(rstd), _I(N), _I(D), _F(eps), _p(self.status(dev)), _st())
            self._rc(rc, "kb_route_pipe_fwd")
        else:       # rows too large for the shared-memory ring: register-resident kernel
            rc = self.lib.kb_route_norm_fwd(arr, _I(S), _p(q), _p(rn_w), _p(n_w), _p(xn), _p(alpha), _p(r), _p(logit),
                                            _p(rstd), _I(N), _I(D), _F(eps), _st())
            self._rc(rc, "kb_route_norm_fwd")
        return xn, (alpha, r, logit, rstd)

    def route_norm_bwd(self, dxn, srcs, q, rn_w, n_w, eps, stats, dsrcs, acc):
        alpha, r, logit, rstd = stats
        S = len(srcs)
        N, D = srcs[0].shape
        dev = dxn.device
        pipe_grid = self.lib.kb_route_pipe_grid(_I(N), _I(S), _I(D), _I(1))
        grid = pipe_grid if pipe_grid > 0 else self.lib.kb_route_bwd_grid(_I(N))
        routing = q is not None
        dnw_part = torch.empty(grid, D, device=dev, dtype=torch.float32)
        dw_part = torch.empty(grid, D, device=dev, dtype=torch.float32) if routing else None
        sa = (_VP * S)(*[s.data_ptr() for s in srcs])
        da = (_VP * S)(*[d.data_ptr() for d in dsrcs])
        mask = sum(1 << i for i, a in enumerate(acc) if a)
        if pipe_grid > 0:
            rc = self.lib.kb_route_pipe_bwd(sa, da, ctypes.c_uint(mask), _I(S), _p(dxn), _p(q), _p(rn_w), _p(n_w),
                                            _p(alpha), _p(r), _p(logit), _p(rstd), _p(dw_part), _p(dnw_part), _I(N),
                                            _I(D), _p(self.status(dev)), _st())
            self._rc(rc, "kb_route_pipe_bwd")
        else:
            rc = self.lib.kb_route_norm_bwd(sa, da, ctypes.c_uint(mask), _I(S), _p(dxn), _p(q), _p(rn_w), _p(n_w),
                                            _p(alpha), _p(r), _p(logit), _p(rstd), _p(dw_part), _p(dnw_part), _I(N),
                                            _I(D), _st())
            self._rc(rc, "kb_route_norm_bwd")
        dn_w = self._colsum(dnw_part)
        if not routing:
            return None, None, dn_w
        dw = self._colsum(dw_part)
        return dw * rn_w.float(), dw * q.float(), dn_w

    # ------------------------------------------------------------------ sampling
    def sample(self, logits, temperature, top_k, top_p, rep_penalty, seeds, counters, seen, slots):
        """Batched device sampler (``csrc/sampler.cu``); per-row parameter sequences go to the device in
        one small copy each."""
        B, V = logits.shape
        dev = logits.device
        f = lambda x: torch.as_tensor(list(x), dtype=torch.float32).to(dev, non_blocking=True)
        i32 = lambda x: torch.as_tensor(list(x), dtype=torch.int32).to(dev, non_blocking=True)
        m = (1 << 63) - 1
        sd = torch.as_tensor([int(x) & m for x in seeds], dtype=torch.int64).to(dev, non_blocking=True)
        out = torch.empty(B, device=dev, dtype=torch.long)
        t, k, p, r, c, sl = f(temperature), i32(top_k), f(top_p), f(rep_penalty), i32(counters), i32(slots)
        if logits.dtype not in (torch.bfloat16, torch.float32) or logits.stride(1) != 1:
            raise KernelError(f"sampler takes bf16/fp32 row-major logits, got {logits.dtype} {logits.stride()}")
        self._call("kb_sample", _p(logits), _I(0 if logits.dtype == torch.bfloat16 else 1), _LL(logits.stride(0)), _I(B),
                   _I(V), _p(t), _p(k), _p(p), _p(r), _p(sd), _p(c), _p(seen), _I(seen.shape[1] if seen is not None else 0),
                   _p(sl), _p(out), _st())
        return out

    # ------------------------------------------------------------------ AttnRes route, blocked form
    def route_blocked_ok(self, S: int, D: int) -> bool:
        return bool(self.lib.kb_route_blocked_ok(_I(S), _I(D)))

    def _fold_w(self, q: torch.Tensor, rn_w: torch.Tensor) -> torch.Tensor:
        w = torch.empty(q.shape, device=q.device, dtype=torch.float32)
        self._call("kb_route_fold_w", _p(q.contiguous()), _p(rn_w.contiguous()), _p(w), _I(q.numel()), _st())
        return w

    @staticmethod
    def _p1_chunk(S: int, D: int) -> int:
        """Queries per phase-1 launch: 8, or 4 where two backward ring stages of 8 would not fit."""
        return 8 if 2 * (S + 8) * (2 * D + 16) <= 200 * 1024 else 4

    def route_p1_fwd(self, srcs, qs, rn_ws, eps):
        S, Q = len(srcs), qs.shape[0]
        N, D = srcs[0].shape
        dev = srcs[0].device
        wf = self._fold_w(qs, rn_ws)
        o = torch.empty(Q, N, D, device=dev, dtype=torch.bfloat16)
        lse = torch.empty(Q, N, device=dev, dtype=torch.float32)
        r = torch.empty(N, S, device=dev, dtype=torch.float32)
        logit = torch.empty(Q, N, S, device=dev, dtype=torch.float32)
        arr = (_VP * S)(*[t.data_ptr() for t in srcs])
        qc = self._p1_chunk(S, D)
        for q0 in range(0, Q, qc):
            n = min(qc, Q - q0)
            self._call("kb_route_p1_fwd", arr, _I(S), _I(n), _p(wf[q0:]), _p(o[q0:]), _p(lse[q0:]), _p(r),
                       _p(logit[q0:]), _I(N), _I(D), _F(eps), _p(self.status(dev)), _st())
        return o, lse, (r, logit, wf)

    def route_p2_fwd(self, o, lse, partial, q, rn_w, n_w, eps):
        N, D = o.shape
        xn = torch.empty(N, D, device=o.device, dtype=torch.bfloat16)
        stats2 = torch.empty(N, 4, device=o.device, dtype=torch.float32)
        w = self._fold_w(q, rn_w) if partial is not None else None
        self._call("kb_route_p2_fwd", _p(o), _p(lse), _p(partial), _p(w), _p(n_w), _p(xn), _p(stats2), _I(N), _I(D),
                   _F(eps), _st())
        return xn, (stats2, w)

    def route_p2_bwd(self, dxn, o, lse, partial, q, rn_w, n_w, eps, stats2, do_out, dlse_out, dpart, dpart_acc):
        stats2, w = stats2
        N, D = o.shape
        dev = o.device
        grid = self.lib.kb_route_blocked_grid(_I(N), _I(2))
        dnw_part = torch.empty(grid, D, device=dev, dtype=torch.float32)
        dw_part = torch.empty(grid, D, device=dev, dtype=torch.float32) if partial is not None else None
        self._call("kb_route_p2_bwd", _p(dxn), _p(o), _p(partial), _p(w), _p(n_w), _p(stats2), _p(do_out), _p(dlse_out),
                   _p(dpart), _I(1 if dpart_acc else 0), _p(dw_part), _p(dnw_part), _I(N), _I(D), _p(self.status(dev)),
                   _st())
        dn_w = self._colsum(dnw_part)
        return (self._colsum(dw_part) if partial is not None else None), dn_w

    def route_p1_bwd(self, srcs, qs, rn_ws, do, dlse, lse, stats, dsrcs, acc):
        r, logit, wf = stats
        S, Q = len(srcs), qs.shape[0]
        N, D = srcs[0].shape
        dev = srcs[0].device
        grid = self.lib.kb_route_blocked_grid(_I(N), _I(1))
        sa = (_VP * S)(*[t.data_ptr() for t in srcs])
        da = (_VP * S)(*[t.data_ptr() for t in dsrcs])
        mask = sum(1 << i for i, a in enumerate(acc) if a)
        dws = torch.empty(Q, D, device=dev, dtype=torch.float32)
        qc = self._p1_chunk(S, D)
        cw = torch.empty(S, N, 8, device=dev, dtype=torch.float32)
        for q0 in range(0, Q, qc):
            n = min(qc, Q - q0)
            self._call("kb_route_p1_bwd", sa, da, ctypes.c_uint(mask), _I(S), _I(n), _p(wf[q0:]), _p(do[q0:]),
                       _p(dlse[q0:]), _p(lse[q0:]), _p(r), _p(logit[q0:]), _p(cw), _I(N), _I(D), _p(self.status(dev)),
                       _st())
            # query gradients: dw_q = sum over tokens and sources of cw * source (streaming pass + column sum)
            part = torch.empty(grid, n * D, device=dev, dtype=torch.float32)
            self._call("kb_route_dw", sa, _I(S), _I(n), _p(cw), _p(part), _I(N), _I(D), _st())
            dws[q0:q0 + n] = self._colsum(part).view(n, D)
            mask = (1 << S) - 1                     # later query chunks add to what the first one wrote
        return dws

    def _colsum(self, part: torch.Tensor) -> torch.Tensor:
        out = torch.empty(part.shape[1], device=part.device, dtype=torch.float32)
        self._rc(self.lib.kb_colsum(_p(part), _p(out), _I(part.shape[0]), _I(part.shape[1]), _st()), "kb_colsum")
        return out

    # ------------------------------------------------------------------ QK-norm + RoPE
    def qknorm_rope_fwd(self, qkv, qw, kw, cos, sin, seq_len, n_q, n_kv, hd, eps, pos_offset=0, positions=None,
                        append=None):
        """``append=(k_pages, v_pages, slots)``: the same launch also writes the rotated keys and the values of
        every token into its cache slot (what ``kv_append`` does as a launch of its own)."""
        N = qkv.shape[0]
        out = torch.empty(N, (n_q + n_kv) * hd, device=qkv.device, dtype=qkv.dtype)
        rstd = torch.empty(N, n_q + n_kv, device=qkv.device, dtype=torch.float32)
        if append is not None:
            k_pages, v_pages, slots = append
            rc = self.lib.kb_qknorm_rope_append(_p(qkv), _p(qw), _p(kw), _p(cos), _p(sin), _p(out), _p(rstd), _I(N),
                                                _I(seq_len), _I(n_q), _I(n_kv), _I(hd), _I(pos_offset), _F(eps),
                                                _p(positions), _p(k_pages), _p(v_pages), _p(slots),
                                                _LL(k_pages.shape[0] * k_pages.shape[-2]), _p(self.status(qkv.device)),
                                                _st())
            self._rc(rc, "kb_qknorm_rope_append")
            return out, rstd
        rc = self.lib.kb_qknorm_rope_fwd(_p(qkv), _p(qw), _p(kw), _p(cos), _p(sin), _p(out), _p(rstd), _I(N),
                                         _I(seq_len), _I(n_q), _I(n_kv), _I(hd), _I(pos_offset), _F(eps), _p(positions),
                                         _st())
        self._rc(rc, "kb_qknorm_rope_fwd")
        return out, rstd

    def qknorm_rope_bwd(self, dqk, qkv, qw, kw, cos, sin, rstd, seq_len, n_q, n_kv, hd, dqkv_out, pos_offset=0):
        N = qkv.shape[0]
        norm = qw is not None
        warps = self.lib.kb_qknorm_grid_warps()
        part = torch.empty(warps, 2 * hd, device=qkv.device, dtype=torch.float32) if norm else None
        rc = self.lib.kb_qknorm_rope_bwd(_p(dqk), _p(qkv), _p(qw), _p(kw), _p(cos), _p(sin), _p(rstd), _p(dqkv_out),
                                         _p(part), _I(N), _I(seq_len), _I(n_q), _I(n_kv), _I(hd), _I(pos_offset), _st())
        self._rc(rc, "kb_qknorm_rope_bwd")
        if not norm:
            return None, None
        dw = self._colsum(part)
        return dw[:hd], dw[hd:]

    # ------------------------------------------------------------------ attention
    def attention_fwd(self, q, k, v, need_grad=True, cu_seqlens=None, max_seqlen=0):
        from .attention import attention_fwd
        return attention_fwd(self, q, k, v, need_grad, cu_seqlens=cu_seqlens, max_seqlen=max_seqlen)

    def attention_bwd(self, do, q, k, v, o, lse, dq_out, dk_out, dv_out):
        from .attention import attention_bwd
        return attention_bwd(self, do, q, k, v, o, lse, dq_out, dk_out, dv_out)

    # ------------------------------------------------------------------ SwiGLU
    def swiglu_fwd(self, gu):
        N, F2 = gu.shape
        act = torch.empty(N, F2 // 2, device=gu.device, dtype=gu.dtype)
        self._rc(self.lib.kb_swiglu_fwd(_p(gu), _p(act), _LL(N), _I(F2 // 2), _st()), "kb_swiglu_fwd")
        return act

    def swiglu_bwd(self, gu, dact, out=None):
        N, F2 = gu.shape
        out = out if out is not None else torch.empty_like(gu)
        self._rc(self.lib.kb_swiglu_bwd(_p(gu), _p(dact), _p(out), _LL(N), _I(F2 // 2), _st()), "kb_swiglu_bwd")
        return out

    # ------------------------------------------------------------------ loss head
    def linear_ce(self, h, w, labels, z_weight, grad_scale, dw, dw_accumulate, chunk=4096, need_grad=True,
                  count=None):
        N, D = h.shape
        V = w.shape[0]
        dev = h.device
        row_ce = torch.empty(N, device=dev, dtype=torch.float32)
        row_z = torch.empty(N, device=dev, dtype=torch.float32)
        nv = (labels >= 0).sum().clamp(min=1).float() if count is None else count.reshape(()).float()
        inv = (1.0 / nv).reshape(1)
        dh = torch.empty_like(h) if need_grad else None
        first = not dw_accumulate
        logits = torch.empty(min(chunk, N), V, device=dev, dtype=h.dtype)
        for s in range(0, N, chunk):
            e = min(N, s + chunk)
            lg = logits[: e - s]
            self.gemm_nt(h[s:e], w, out=lg)
            rc = self.lib.kb_ce_zloss(_p(lg), _p(labels[s:e]), _p(row_ce[s:e]), _p(row_z[s:e]), _p(inv),
                                      _F(z_weight), _F(grad_scale), _I(e - s), _I(V), _I(int(need_grad)),
                                      _p(self.status(dev)), _st())
            self._rc(rc, "kb_ce_zloss")
            if need_grad:
                self.gemm_nn(lg, w, out=dh[s:e])
                if dw is not None:
                    self.gemm_tn(lg, h[s:e], out=dw, accumulate=not first)
                    first = False
        sums = torch.empty(2, device=dev, dtype=torch.float32)
        self._rc(self.lib.kb_sum_f32(_p(row_ce), _I(N), _p(sums[0:1]), _st()), "kb_sum_f32")
        self._rc(self.lib.kb_sum_f32(_p(row_z), _I(N), _p(sums[1:2]), _st()), "kb_sum_f32")
        return sums[0] * inv[0], sums[1] * (z_weight * inv[0]), dh

    # ------------------------------------------------------------------ embedding
    def embedding_fwd(self, ids, w):
        N, D = ids.numel(), w.shape[1]
        out = torch.empty(N, D, device=w.device, dtype=w.dtype)
        self._rc(self.lib.kb_embedding_fwd(_p(ids), _p(w), _p(out), _I(N), _I(D), _I(w.shape[0]),
                                           _p(self.status(w.device)), _st()), "kb_embedding_fwd")
        return out

    def embedding_bwd(self, dout, ids, dw):
        self._rc(self.lib.kb_embedding_bwd(_p(ids), _p(dout), _p(dw), _I(ids.numel()), _I(dw.shape[1]), _I(dw.shape[0]),
                                           _p(self.status(dw.device)), _st()), "kb_embedding_bwd")

    # ------------------------------------------------------------------ optimizer math
    def sumsq(self, x, out: Optional[torch.Tensor] = None, accumulate: bool = False):
        dt = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}[x.dtype]
        partial = torch.empty(1024, device=x.device, dtype=torch.float32)
        res = out if out is not None else torch.empty(1, device=x.device, dtype=torch.float32)
        self._rc(self.lib.kb_sumsq(_p(x), _LL(x.numel()), _I(dt), _p(partial), _p(res), _I(int(accumulate)), _st()),
                 "kb_sumsq")
        self.launches += 1
        return res[0] if out is None else res

    def adamw_step(self, p, g, m, v, step, lr, b1, b2, eps, wd, gscale):
        gs = gscale.reshape(1).float() if isinstance(gscale, torch.Tensor) else None
        if gs is None and gscale != 1.0:
            gs = torch.full((1,), float(gscale), device=p.device)
        self._rc(self.lib.kb_adamw(_p(p), _p(g), _p(m), _p(v), _LL(p.numel()), _p(gs), _F(lr), _F(b1), _F(b2),
                                   _F(eps), _F(wd), _I(step), _st()), "kb_adamw")

    def muon_momentum(self, g, buf, momentum, nesterov, gscale):
        gs = gscale.reshape(1).float() if isinstance(gscale, torch.Tensor) else None
        x = torch.empty(g.shape, device=g.device, dtype=torch.float16)
        partial = torch.empty(1024, device=g.device, dtype=torch.float32)
        sq = torch.empty(1, device=g.device, dtype=torch.float32)
        self._rc(self.lib.kb_muon_momentum(_p(g), _p(buf), _p(x), _LL(g.numel()), _p(gs), _F(momentum),
                                           _I(int(nesterov)), _p(partial), _p(sq), _st()), "kb_muon_momentum")
        self.launches += 1
        return x, sq

    def ns_normalize(self, x, sumsq):
        self._rc(self.lib.kb_ns_normalize(_p(x), _LL(x.numel()), _p(sumsq.reshape(1)), _st()), "kb_ns_normalize")
        return x

    def ns_iteration(self, x, a, b, c):
        """``A = X X^T``, ``B = bA + cA^2``, ``X' = aX + BX``: three tcgen05 GEMMs with the polynomial
        terms fused into their epilogues.  ``A`` and ``A^2`` are symmetric, so only the tiles on and
        above the diagonal are computed and then mirrored."""
        R, C = x.shape[-2], x.shape[-1]
        batch = x.shape[0] if x.ndim == 3 else 1
        sym = self.gemm_2cta and R >= 512 and x.element_size() == 2
        A = self._gemm(x, x, R, R, C, False, False, batch=batch, sym_upper=sym)
        # aX + BX = (B + aI) X: the identity term goes onto B's diagonal in the epilogue that produces B,
        # so the last (largest) product needs no addend
        B = self._gemm(A, A, R, R, R, False, False, cin=A, alpha=c, beta=b, batch=batch, sym_upper=sym, diag=a)
        if self.mn_major:
            return self._gemm(B, x, R, C, R, False, True, batch=batch)
        xt = self.transpose(x) if x.ndim == 2 else x.transpose(-1, -2).contiguous()
        return self._gemm(B, xt, R, C, R, False, False, batch=batch)

    def muon_apply(self, p, orth, lr, wd, scale, transposed):
        R, C = p.shape
        self._rc(self.lib.kb_muon_apply(_p(p), _p(orth), _I(R), _I(C), _F(lr), _F(wd), _F(scale),
                                        _I(int(transposed)), _st()), "kb_muon_apply")

    def transpose(self, x):
        assert x.ndim == 2 and x.is_contiguous() and x.element_size() == 2
        out = torch.empty(x.shape[1], x.shape[0], device=x.device, dtype=x.dtype)
        self._rc(self.lib.kb_transpose16(_p(x), _p(out), _I(x.shape[0]), _I(x.shape[1]), _st()), "kb_transpose16")
        return out

    # ------------------------------------------------------------------ serving
    def kv_append(self, k, v, k_pages, v_pages, slots):
        """Copy rows ``k[n], v[n]`` (``[N, n_kv*hd]`` views) into cache slot ``slots[n]`` (page*16 + offset)."""
        N, row = k.shape
        self._rc(self.lib.kb_kv_append(_p(k), _p(v), _LL(k.stride(0)), _LL(v.stride(0)), _p(k_pages), _p(v_pages),
                                       _p(slots), _I(N), _I(row), _I(k_pages.shape[-1]),
                                       _LL(k_pages.shape[0] * k_pages.shape[-2]), _p(self.status(k.device)), _st()),
                 "kb_kv_append")

    def paged_decode_attention(self, q, k_pages, v_pages, page_table, ctx_lens, max_ctx, n_q, n_kv, hd, split=512):
        """``q[B, n_q*hd]`` (one new token per request) against the paged cache; returns ``[B, n_q*hd]``."""
        B = q.shape[0]
        nsplit = (max_ctx + split - 1) // split
        G = n_q // n_kv
        part_o = torch.empty(B * n_kv * nsplit * G * hd, device=q.device, dtype=torch.float32)
        part_ml = torch.empty(B * n_kv * nsplit * G * 2, device=q.device, dtype=torch.float32)
        out = torch.empty(B, n_q * hd, device=q.device, dtype=q.dtype)
        # election counters of the in-kernel merge: zero once, left at zero by every call
        key = (q.device.index, B * n_kv)
        counters = self._merge_counters.get(key)
        if counters is None:
            counters = self._merge_counters[key] = torch.zeros(B * n_kv, device=q.device, dtype=torch.int32)
        rc = self.lib.kb_paged_decode_merged(_p(q), _LL(q.stride(0)), _p(k_pages), _p(v_pages), _p(page_table),
                                             _I(page_table.shape[1]), _p(ctx_lens), _I(B), _I(n_q), _I(n_kv), _I(hd),
                                             _I(max_ctx), _I(split), _F(1.0 / math.sqrt(hd)), _p(part_o), _p(part_ml),
                                             _p(out), _LL(out.stride(0)), _I(k_pages.shape[0]),
                                             _p(counters if self.decode_merge_fused else None), _st())
        self._rc(rc, "kb_paged_decode")
        self.launches += 1
        return out

    def argmax(self, logits):
        out = torch.empty(logits.shape[0], device=logits.device, dtype=torch.long)
        self._rc(self.lib.kb_argmax(_p(logits), _LL(logits.stride(0)), _I(logits.shape[0]), _I(logits.shape[1]),
                                    _p(out), _st()), "kb_argmax")
        return out
