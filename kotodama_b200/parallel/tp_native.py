"""Tensor + sequence parallelism whose collectives run inside our own kernels over NVLink.

``TensorParallelComm`` calls the library (all-gather, reduce-scatter) around plain GEMMs.  This
strategy replaces those pairs by fused kernels on symmetric memory:

* **all-gather -> GEMM** (column-parallel projections, and the backward of row-parallel ones):
  ``kb_ag_push`` stores this rank's activation shard into every peer's staging buffer and raises
  the shard's ready flag; ``kb_gemm_ag`` is the tcgen05 GEMM whose TMA producer waits (bounded)
  for a shard's flag only when it reaches the first tile of that shard, and visits its own shard
  first - the transfer of shard *s+1* overlaps the math on shard *s*;
* **GEMM -> reduce-scatter** (row-parallel projections, and the data gradient of column-parallel
  ones): ``kb_gemm_rs`` stores each finished output tile straight into the owner rank's slab while
  the remaining tiles are still being computed and counts arrivals on the owner;
  ``kb_rs_reduce`` waits for the arrivals, sums the slabs in fp32, adds the residual and frees
  the slabs for the call after next;
* the weight gradient of a column-parallel projection gathers along K: same kernel, waits per
  k-block.

Staging buffers and slabs are double-buffered; a buffer is reused only after every peer reported
(through a flag) that it finished reading the call that used it two calls ago.  All waits are
bounded and report through the ops status word.

The reference has no counterpart: its tensor parallelism all-reduces replicated activations
(``src/training/tensor_parallel.py:31-65``).
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

import torch
import torch.distributed as dist

from .tp import TensorParallelComm

_VP, _I, _LL, _F, _D = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double

# slots of the per-rank sync array (8 ints each, indexed by source rank)
_AG_READY, _AG_DONE, _RS_CNT, _RS_DONE, _SMALL = 0, 2, 3, 5, 6      # AG_READY and RS_CNT take two slots (parity)
_N_SLOTS = 8
_BM, _BK = 128, 64


class FusedTensorParallelComm(TensorParallelComm):
    WAIT_LIMIT_S = 20.0

    def __init__(self, tp_group: Any, dp_group: Any = None, max_ctas: int = 64) -> None:
        super().__init__(tp_group, dp_group, sequence_parallel=True)
        import torch.distributed._symmetric_memory as symm_mem
        self.symm_mem = symm_mem
        self.max_ctas = max_ctas
        self.ag_calls = 0
        self.rs_calls = 0
        self._bufs: dict = {}
        self.fused_calls = 0
        self.fallback_calls = 0
        # KB_TP_AG_PAIR=0 keeps the coupled products on the 1-CTA kernel (tuning / comparison)
        self.pair_gemm = os.environ.get("KB_TP_AG_PAIR", "1") != "0"

    # ------------------------------------------------------------------ set-up
    def attach(self, engine: Any) -> None:
        super().attach(engine)
        self.setup(engine.device, engine.ops)

    def setup(self, device: Any, ops: Any) -> None:
        """Symmetric-memory set-up (collective over the TP group).  ``attach`` calls it; the kernel
        benchmarks call it directly, without an engine."""
        self._ops = ops
        if hasattr(self, "lib"):
            return
        from ..ops import _build
        self.lib = _build.load()
        dev = self._device = torch.device(device)
        self.sync = self.symm_mem.empty(_N_SLOTS * 8, dtype=torch.int32, device=dev)
        self.sync.zero_()
        h = self.symm_mem.rendezvous(self.sync, self.tp_group)
        self._h = [h]
        self.sync_ptrs = [int(p) for p in h.buffer_ptrs]
        self.counters = torch.zeros(4, device=dev, dtype=torch.int32)     # last-block elections
        # packed small all-reduce (loss terms, squared gradient norm): values [2 parities][8 ranks][8 floats]
        self.small_vals = self.symm_mem.empty(2 * 8 * 8, dtype=torch.float32, device=dev)
        self.small_vals.zero_()
        h_s = self.symm_mem.rendezvous(self.small_vals, self.tp_group)
        self._h.append(h_s)
        self.small_ptrs = [int(p) for p in h_s.buffer_ptrs]
        self.small_calls = 0
        self.side = torch.cuda.Stream(device=dev)
        torch.cuda.synchronize()
        dist.barrier(group=self.tp_group)

    def _small_allreduce(self, t: torch.Tensor) -> torch.Tensor:
        """Sum of a few floats over the TP group inside one kernel (no library collective)."""
        n = t.numel()
        if not (hasattr(self, "small_ptrs") and t.is_cuda and n <= 8):
            dist.all_reduce(t, group=self.tp_group)
            return t
        src = t.reshape(-1).float().contiguous()
        out = torch.empty_like(src)
        self.small_calls += 1
        rc = self.lib.kb_packed_allreduce(self._arr(self.small_ptrs), self._arr(self.sync_ptrs), _I(self.tp_size),
                                          _I(self.tp_rank), _I(_SMALL), _I(self.small_calls), _VP(src.data_ptr()),
                                          _VP(out.data_ptr()), _I(n), _D(self.WAIT_LIMIT_S), self._status(), self._st())
        self._ck(rc, "kb_packed_allreduce")
        return out.reshape(t.shape).to(t.dtype)

    def loss_reduce(self, t: torch.Tensor) -> torch.Tensor:
        return self._small_allreduce(t)

    def grad_sumsq(self, ops) -> torch.Tensor:
        ar = self.engine.arena
        sharded = self._small_allreduce(ops.sumsq(ar.grads[:ar.muon_end]).reshape(1).clone())
        lo, hi = ar.adamw_range()
        return (sharded + ops.sumsq(ar.grads[lo:hi]).reshape(1))[0]

    def _buffer(self, kind: str, elems: int) -> tuple[torch.Tensor, list[int]]:
        """Symmetric buffer of at least ``elems`` bf16 elements per parity (2 parities).  Grows by
        re-allocation; every rank calls this with the same sizes in the same order."""
        cur = self._bufs.get(kind)
        if cur is None or cur[0].numel() < 2 * elems:
            torch.cuda.synchronize()
            dist.barrier(group=self.tp_group)      # nobody may still be writing into the old buffer
            t = self.symm_mem.empty(2 * elems, dtype=torch.bfloat16, device=self._device)
            h = self.symm_mem.rendezvous(t, self.tp_group)
            self._h.append(h)
            cur = (t, [int(p) for p in h.buffer_ptrs], elems)
            self._bufs[kind] = cur
            dist.barrier(group=self.tp_group)
        return cur

    def _status(self) -> _VP:
        return _VP(self._ops.status(self._device).data_ptr())

    @staticmethod
    def _st() -> _VP:
        return _VP(torch.cuda.current_stream().cuda_stream)

    def _ck(self, rc: int, what: str) -> None:
        self._ops.launches += 1
        if rc != 0:
            raise RuntimeError(f"{what}: launcher returned {rc}")

    def _arr(self, vals) -> Any:
        return (_VP * 8)(*([int(v) for v in vals] + [0] * (8 - len(vals))))

    def _sync_addr(self, peer: int, slot: int, idx: int) -> int:
        return self.sync_ptrs[peer] + 4 * (slot * 8 + idx)

    # ------------------------------------------------------------------ all-gather side
    def _usable(self, x: torch.Tensor) -> bool:
        return (x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape[0] % _BM == 0
                and x.shape[-1] % 8 == 0 and hasattr(self, "lib"))

    def _push(self, x: torch.Tensor) -> tuple[torch.Tensor, int, int]:
        """Start the all-gather of ``x`` ([rows, width]); returns (gathered view, call number, parity)."""
        rows, width = x.shape
        W, r = self.tp_size, self.tp_rank
        self.ag_calls += 1
        c, par = self.ag_calls, self.ag_calls & 1
        elems = W * rows * width
        buf, ptrs, cap = self._buffer("ag", elems)
        base_off = par * cap                      # element offset of this parity's buffer
        stage = [ptrs[q] + 2 * (base_off + r * rows * width) for q in range(W)]
        ready = [self._sync_addr(q, _AG_READY + par, r) for q in range(W)]
        done_local = self.sync.data_ptr() + 4 * (_AG_DONE * 8)
        main = torch.cuda.current_stream()

        def push(first: int, count: int, counter: int, stream) -> None:
            rc = self.lib.kb_ag_push(_VP(x.data_ptr()), _LL(rows * width), self._arr(stage), self._arr(ready), _I(W),
                                     _I(first), _I(count), _I(c), _VP(done_local), _I(max(c - 2, 0)),
                                     _VP(self.counters[counter:counter + 1].data_ptr()), _D(self.WAIT_LIMIT_S),
                                     self._status(), _I(self.max_ctas), _VP(stream.cuda_stream))
            self._ck(rc, "kb_ag_push")

        # own shard: a local copy on the compute stream, so the GEMM (which starts on its own shard)
        # never waits for the network; peers: from the side stream, under the GEMM's first tiles
        push(r, 1, 0, main)
        if W > 1:
            self.side.wait_stream(main)
            push((r + 1) % W, W - 1, 2, self.side)
            self._side_busy = True
        view = buf[base_off: base_off + elems].view(W * rows, width)
        return view, c, par

    def _ag_done(self, c: int) -> None:
        """Tell every peer that this rank has finished reading the staging buffer of call ``c``."""
        if getattr(self, "_side_busy", False):
            torch.cuda.current_stream().wait_stream(self.side)     # the pushed tensor may be freed after this
            self._side_busy = False
        rc = self.lib.kb_flag_signal(self._arr(self.sync_ptrs), _I(self.tp_size), _I(self.tp_rank), _I(_AG_DONE),
                                     _I(c), self._st())
        self._ck(rc, "kb_flag_signal")

    def _gemm_ag(self, a, b, out, M, N, K, lda, ldb, a_mn, b_mn, par, c, rows, dim, cin=None, beta=0.0) -> None:
        flags = self.sync.data_ptr() + 4 * ((_AG_READY + par) * 8)
        # the CTA-pair kernel (wider tiles, faster) takes shards that are whole 256-row tiles
        pair = self.pair_gemm and (rows % (2 * _BM) == 0 if dim == 0 else rows % _BK == 0)
        fn = self.lib.kb_gemm_2cta_ag if pair else self.lib.kb_gemm_ag
        rc = fn(_VP(a.data_ptr()), _VP(b.data_ptr()), _VP(out.data_ptr()),
                                 _VP(cin.data_ptr() if cin is not None else None), _I(M), _I(N), _I(K), _LL(lda),
                                 _LL(ldb), _LL(N), _I(a_mn), _I(b_mn), _F(1.0), _F(beta), _VP(flags), _I(c),
                                 _I(rows), _I(dim), _I(self.tp_rank), _D(self.WAIT_LIMIT_S), self._status(),
                                 self._st())
        self._ck(rc, "kb_gemm_2cta_ag" if pair else "kb_gemm_ag")

    def col_linear(self, ops, x, w):
        if not (isinstance(w, torch.Tensor) and self._usable(x) and w.dtype == torch.bfloat16 and w.is_contiguous()):
            self.fallback_calls += 1
            return super().col_linear(ops, x, w)
        rows, K = x.shape
        gathered, c, par = self._push(x)
        N = w.shape[0]
        out = torch.empty(gathered.shape[0], N, device=x.device, dtype=x.dtype)
        self._gemm_ag(gathered, w, out, gathered.shape[0], N, K, K, K, 0, 0, par, c, rows, 0)
        self._ag_done(c)
        self.fused_calls += 1
        return out

    def row_linear_bwd(self, ops, dy, w, x_saved, g_out, accumulate: bool):
        if not (isinstance(w, torch.Tensor) and self._usable(dy) and w.dtype == torch.bfloat16 and w.is_contiguous()):
            self.fallback_calls += 1
            return super().row_linear_bwd(ops, dy, w, x_saved, g_out, accumulate)
        rows, D = dy.shape
        gathered, c, par = self._push(dy)
        M, N = gathered.shape[0], w.shape[1]                  # w is [D, F/tp]: dx = dy_full @ w
        dx = torch.empty(M, N, device=dy.device, dtype=dy.dtype)
        self._gemm_ag(gathered, w, dx, M, N, D, D, N, 0, 1, par, c, rows, 0)
        # every shard has landed once the product above is done: the weight gradient reads the
        # same staging buffer with the ordinary GEMM
        ops.gemm_tn(gathered, x_saved, out=g_out, accumulate=accumulate)
        self._ag_done(c)
        self.fused_calls += 1
        return dx

    # ------------------------------------------------------------------ reduce-scatter side
    def _gemm_rs(self, a, b, M, N, K, lda, ldb, a_mn, b_mn, residual) -> torch.Tensor:
        W, r = self.tp_size, self.tp_rank
        rows = M // W
        self.rs_calls += 1
        c, par = self.rs_calls, self.rs_calls & 1
        slab = rows * N
        buf, ptrs, cap = self._buffer("rs", W * slab)
        base_off = par * cap
        if c > 2:       # the owners must have reduced the call that used these slabs before
            rc = self.lib.kb_flag_wait(_VP(self.sync.data_ptr()), _I(W), _I(_RS_DONE), _I(c - 2),
                                       _D(self.WAIT_LIMIT_S), self._status(), self._st())
            self._ck(rc, "kb_flag_wait")
        outs = [ptrs[o] + 2 * (base_off + r * slab) for o in range(W)]
        cnts = [self._sync_addr(o, _RS_CNT + par, r) for o in range(W)]
        pair = self.pair_gemm and rows % (2 * _BM) == 0
        fn = self.lib.kb_gemm_2cta_rs if pair else self.lib.kb_gemm_rs
        rc = fn(_VP(a.data_ptr()), _VP(b.data_ptr()), _I(M), _I(N), _I(K), _LL(lda), _LL(ldb), _LL(N),
                _I(a_mn), _I(b_mn), _F(1.0), self._arr(outs), self._arr(cnts), _I(W), _I(r),
                _I(rows), self._status(), self._st())
        self._ck(rc, "kb_gemm_2cta_rs" if pair else "kb_gemm_rs")
        expected = int(self.lib.kb_gemm_2cta_rs_arrivals(_I(M), _I(N), _I(rows)) if pair
                       else self.lib.kb_gemm_rs_arrivals(_I(N), _I(rows)))
        out = torch.empty(rows, N, device=a.device, dtype=torch.bfloat16)
        done = [self._sync_addr(q, _RS_DONE, r) for q in range(W)]
        rc = self.lib.kb_rs_reduce(_VP(buf.data_ptr() + 2 * base_off), _LL(slab),
                                   _VP(self.sync.data_ptr() + 4 * ((_RS_CNT + par) * 8)), _I(expected),
                                   _I(W), _VP(residual.data_ptr() if residual is not None else None),
                                   _VP(out.data_ptr()), self._arr(done), _I(c), _VP(self.counters[1:2].data_ptr()),
                                   _D(self.WAIT_LIMIT_S), self._status(), _I(4 * self.max_ctas), self._st())
        self._ck(rc, "kb_rs_reduce")
        return out

    def _rs_usable(self, x: torch.Tensor, w: torch.Tensor) -> bool:
        return (isinstance(w, torch.Tensor) and x.is_cuda and x.dtype == torch.bfloat16 and x.is_contiguous()
                and w.is_contiguous() and w.dtype == torch.bfloat16 and x.shape[0] % (self.tp_size * _BM) == 0 and hasattr(self, "lib"))

    def row_linear(self, ops, x, w, residual=None):
        if not self._rs_usable(x, w) or w.shape[0] % 8 or (residual is not None and not residual.is_contiguous()):
            self.fallback_calls += 1
            return super().row_linear(ops, x, w, residual=residual)
        M, K = x.shape
        self.fused_calls += 1
        return self._gemm_rs(x, w, M, w.shape[0], K, K, K, 0, 0, residual)

    def col_linear_bwd(self, ops, dy, w, x, g_out, accumulate: bool):
        ok = (self._usable(x) and self._rs_usable(dy, w) and g_out.is_contiguous() and x.shape[0] % _BK == 0
              and w.shape[1] % 8 == 0)
        if not ok:
            self.fallback_calls += 1
            return super().col_linear_bwd(ops, dy, w, x, g_out, accumulate)
        rows, D = x.shape
        gathered, c, par = self._push(x)
        Ktok, Nout = dy.shape                                   # dy [tokens, F'/tp]; g_out [F'/tp, D]
        self._gemm_ag(dy, gathered, g_out, Nout, D, Ktok, Nout, D, 1, 1, par, c, rows, 1,
                      cin=g_out if accumulate else None, beta=1.0 if accumulate else 0.0)
        self._ag_done(c)
        self.fused_calls += 1
        # data gradient: dy [tokens, F'/tp] @ w [F'/tp, D] -> reduce-scatter over tokens
        return self._gemm_rs(dy, w, Ktok, D, Nout, Nout, D, 0, 1, None)
