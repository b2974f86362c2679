"""Data-parallel communication issued from our own kernels over NVLink peer memory.

The parameter and gradient arenas are allocated in symmetric memory (every rank maps every
peer's arena).  Per optimizer step:

1. when the backward of layer ``i`` is done, the rank raises flag ``i`` on every peer (compute
   stream) and queues, on the communication stream, a bounded wait for all ranks' flag ``i``
   followed by *reduce-to-owner* kernels: the owner of each matrix sums that matrix's gradient
   over all ranks (fp32), applies ``1/world`` and stores bf16 into its own gradient arena.  This
   overlaps with the backward of layer ``i-1``;
2. embeddings / norms / queries (every rank updates them) use a two-shot all-reduce:
   each rank reduces one slice and stores it into every rank's arena;
3. the global gradient norm is a one-float all-reduce (each rank contributes the squares of the
   matrices it owns, rank 0 adds the replicated range);
4. Muon runs only on the owner; its last kernel writes the new parameter into every rank's arena
   (the all-gather is the parameter write);
5. a final flag barrier lets no rank start the next forward before all parameters have landed.

Waits are bounded on the device (status word, checked by the host at step end).  The reference
does stock DDP all-reduce plus Newton-Schulz replicated on every rank
(``src/training/train.py:328-340``, ``src/training/muon.py:255-351``).
"""
from __future__ import annotations

import ctypes
from typing import Any

import torch
import torch.distributed as dist

from .comm import LocalComm

_VP, _I, _LL, _F, _D = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_float, ctypes.c_double


class NativeComm(LocalComm):
    WAIT_LIMIT_S = 20.0

    def __init__(self, group: Any = None, distributed_muon: bool = True, max_ctas: int = 32) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        if not (dist.is_available() and dist.is_initialized()):
            raise RuntimeError("NativeComm needs an initialised process group for the rendezvous")
        self.symm_mem = symm_mem
        self.group = group or dist.group.WORLD
        self.world = dist.get_world_size(self.group)
        self.rank = dist.get_rank(self.group)
        if self.world > 8:
            raise RuntimeError("NativeComm covers one NVSwitch domain of at most 8 GPUs")
        self.dp_size = self.world
        self.distributed_muon = distributed_muon
        self.max_ctas = max_ctas
        self.epoch = 0
        self._handles: list = []
        self._arenas: list[torch.Tensor] = []
        self.comm_stream = None

    # ---------------------------------------------------------------- allocation
    def allocator(self, device: torch.device, dtype: torch.dtype):
        def alloc(n: int) -> torch.Tensor:
            t = self.symm_mem.empty(n, dtype=dtype, device=device)
            t.zero_()
            self._arenas.append(t)
            return t
        return alloc

    def _ptr_array(self, ptrs) -> Any:
        return (_VP * self.world)(*[int(p) for p in ptrs])

    def attach(self, engine: Any) -> None:
        first = not hasattr(self, "engine")
        self.engine = engine
        ar = engine.arena
        if first:
            from ..ops import _build
            self.lib = _build.load()
            dev = engine.device
            self.comm_stream = torch.cuda.Stream(device=dev)
            h_p = self.symm_mem.rendezvous(ar.params, self.group)
            h_g = self.symm_mem.rendezvous(ar.grads, self.group)
            self.n_slots = engine.cfg.num_layers + 8
            self.flags = self.symm_mem.empty(self.n_slots * 8, dtype=torch.int32, device=dev)
            self.flags.zero_()
            self.vals = self.symm_mem.empty(16, dtype=torch.float32, device=dev)
            self.vals.zero_()
            h_f = self.symm_mem.rendezvous(self.flags, self.group)
            h_v = self.symm_mem.rendezvous(self.vals, self.group)
            self._handles = [h_p, h_g, h_f, h_v]
            self.p_ptrs, self.g_ptrs = self._ptr_array(h_p.buffer_ptrs), self._ptr_array(h_g.buffer_ptrs)
            self.f_ptrs, self.v_ptrs = self._ptr_array(h_f.buffer_ptrs), self._ptr_array(h_v.buffer_ptrs)
            self.sq_partial = torch.zeros(1, device=dev, dtype=torch.float32)
            self.sq_total = torch.zeros(1, device=dev, dtype=torch.float32)
            self._by_layer: dict[int, list] = {}
            for s in ar.muon_slots():
                self._by_layer.setdefault(s.layer, []).append(s)
            torch.cuda.synchronize()
            dist.barrier(group=self.group)
        # identical starting weights everywhere (cold path: library broadcast)
        dist.broadcast(ar.params, src=dist.get_global_rank(self.group, 0), group=self.group)
        torch.cuda.synchronize()
        dist.barrier(group=self.group)

    def _check(self, rc: int, what: str) -> None:
        self.engine.ops.launches += 1
        if rc != 0:
            raise RuntimeError(f"{what}: launcher returned {rc}")

    def _status(self) -> _VP:
        return _VP(self.engine.ops.status(self.engine.device).data_ptr())

    def _stream(self, s=None) -> _VP:
        return _VP((s or torch.cuda.current_stream()).cuda_stream)

    # ---------------------------------------------------------------- gradient reduction
    def begin_step(self) -> None:
        self.epoch += 1

    def _signal(self, slot: int) -> None:
        self._check(self.lib.kb_flag_signal(self.f_ptrs, _I(self.world), _I(self.rank), _I(slot), _I(self.epoch),
                                            self._stream()), "kb_flag_signal")

    def _wait(self, slot: int, stream) -> None:
        if stream is not None and stream != torch.cuda.current_stream():
            # the wait must not start before this rank itself has reached the point of the signal:
            # a wait kernel that spins on the side stream while the forward still runs was measured
            # to slow the concurrent GEMMs by 1.5x at 4 and 8 ranks
            stream.wait_stream(torch.cuda.current_stream())
        self._check(self.lib.kb_flag_wait(_VP(self.flags.data_ptr()), _I(self.world), _I(slot), _I(self.epoch),
                                          _D(self.WAIT_LIMIT_S), self._status(), self._stream(stream)), "kb_flag_wait")

    def layer_grads_ready(self, layer: int) -> None:
        if self._first_of_step:
            self.begin_step()
            self._first_of_step = False
        slot = layer if layer >= 0 else self.engine.cfg.num_layers + 1
        self._signal(slot)
        cs = self.comm_stream
        self._wait(slot, cs)                 # starts after our own signal, then polls for the peers'
        ar = self.engine.arena
        for s in self._by_layer.get(layer, []):
            if self.distributed_muon and s.owner != self.rank:
                continue
            out = ar.grads[s.offset:s.offset + s.numel]
            if self.distributed_muon:
                rc = self.lib.kb_reduce_to_owner(self.g_ptrs, _I(self.world), _LL(s.offset), _LL(s.numel),
                                                 _F(1.0), _VP(out.data_ptr()), _I(self.max_ctas), self._stream(cs))
                self._check(rc, "kb_reduce_to_owner")
            else:
                rc = self.lib.kb_allreduce_slices(self.g_ptrs, _I(self.world), _I(self.rank), _LL(s.offset),
                                                  _LL(s.numel), _F(1.0), _I(self.max_ctas), self._stream(cs))
                self._check(rc, "kb_allreduce_slices")

    _first_of_step = True

    def small_grads_ready(self) -> None:
        if self._first_of_step:
            self.begin_step()
            self._first_of_step = False
        L = self.engine.cfg.num_layers
        self._signal(L)
        cs = self.comm_stream
        self._wait(L, cs)
        lo, hi = self.engine.arena.adamw_range()
        rc = self.lib.kb_allreduce_slices(self.g_ptrs, _I(self.world), _I(self.rank), _LL(lo), _LL(hi - lo), _F(1.0),
                                          _I(self.max_ctas), self._stream(cs))
        self._check(rc, "kb_allreduce_slices")
        if -1 in self._by_layer:
            self.layer_grads_ready(-1)
        # every rank's slice (and, without owner-computes, every matrix) must have landed
        # everywhere before anyone reads: signal after our writes, wait for all
        self._check(self.lib.kb_flag_signal(self.f_ptrs, _I(self.world), _I(self.rank), _I(L + 2), _I(self.epoch),
                                            self._stream(cs)), "kb_flag_signal")
        self._wait(L + 2, cs)

    def finish_grad_reduce(self) -> None:
        torch.cuda.current_stream().wait_stream(self.comm_stream)
        self._first_of_step = True

    def grad_sumsq(self, ops) -> torch.Tensor:
        ar = self.engine.arena
        self.sq_partial.zero_()
        if self.distributed_muon:
            for s in ar.muon_slots():
                if s.owner == self.rank:
                    ops.sumsq(ar.grads[s.offset:s.offset + s.numel], out=self.sq_partial, accumulate=True)
            if self.rank == 0:
                lo, hi = ar.adamw_range()
                ops.sumsq(ar.grads[lo:hi], out=self.sq_partial, accumulate=True)
        else:
            if self.rank == 0:
                ops.sumsq(ar.grads, out=self.sq_partial, accumulate=True)
        L = self.engine.cfg.num_layers
        rc = self.lib.kb_scalar_allreduce(self.v_ptrs, self.f_ptrs, _I(self.world), _I(self.rank), _I(L + 3),
                                          _I(self.epoch), _VP(self.sq_partial.data_ptr()),
                                          _VP(self.sq_total.data_ptr()), _D(self.WAIT_LIMIT_S), self._status(),
                                          self._stream())
        self._check(rc, "kb_scalar_allreduce")
        return self.sq_total[0]

    # ---------------------------------------------------------------- Muon parameter write
    def muon_apply(self, ops, slot, orth: torch.Tensor, lr: float, wd: float, scale: float, transposed: bool) -> None:
        R, C = slot.shape
        rc = self.lib.kb_muon_apply_bcast(self.p_ptrs, _I(self.world), _I(self.rank), _LL(slot.offset),
                                          _VP(orth.data_ptr()), _I(R), _I(C), _F(lr), _F(wd), _F(scale),
                                          _I(int(transposed)), self._stream())
        self._check(rc, "kb_muon_apply_bcast")

    def finish_param_publish(self) -> None:
        L = self.engine.cfg.num_layers
        rc = self.lib.kb_scalar_allreduce(self.v_ptrs, self.f_ptrs, _I(self.world), _I(self.rank), _I(L + 4),
                                          _I(self.epoch), _VP(None), _VP(None), _D(self.WAIT_LIMIT_S), self._status(),
                                          self._stream())
        self._check(rc, "kb_scalar_allreduce")

    def gather_momentum(self, slot, buf):
        if not self.distributed_muon:
            return buf
        if buf is None:
            buf = torch.zeros(slot.shape, device=self.engine.device, dtype=self.engine.dtype)
        out = buf.clone()
        dist.broadcast(out, src=dist.get_global_rank(self.group, slot.owner), group=self.group)
        return out

    def barrier(self) -> None:
        dist.barrier(group=self.group)

    def all_reduce_max(self, value: float) -> float:
        t = torch.tensor([value], dtype=torch.float64, device=self.engine.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())
