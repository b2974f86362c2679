"""Tensor-parallel serving: one process per GPU, every rank runs the same ``ServingEngine`` on its
shard of the heads / MLP columns and of the paged KV cache (KV heads are sharded with the
attention heads), and the two row-parallel projections of each layer are all-reduced.

* ``ServeTP`` is the helper the engine calls: ``prepare_model`` shards the projections,
  ``row_linear`` is GEMM -> all-reduce (+ residual).  On CUDA the all-reduce is our own
  kernel over symmetric memory - ``kb_allreduce_multimem`` (the sum is done inside NVSwitch by
  ``multimem.ld_reduce`` on this job's own symmetric buffers) where the buffers have a multicast
  mapping, else ``kb_allreduce_push`` (plain peer stores): the call counter lives in device
  memory, so decode steps that contain it can be captured in a CUDA graph and replayed; activations
  larger than the receive slots (long prefills) and the CPU path use the library all-reduce.
* ranks stay in lock-step by construction: rank 0 owns the request queue, ``TPLeader.step``
  broadcasts a fixed-size header tensor (and, only when something was admitted or cancelled since
  the last step, a byte tensor describing it) and then every rank executes the same
  ``engine.step()``; sampling is a function of the all-reduced (bitwise identical) logits and of
  per-request seeds, so all ranks pick the same tokens.  ``run_follower`` is the loop of ranks > 0.

The reference serves one request at a time on one GPU (``serve.py:322-391``).
"""
from __future__ import annotations

import ctypes
import dataclasses
import json
import os
from typing import Any, Optional

import torch
import torch.distributed as dist

_VP, _I, _LL, _D = ctypes.c_void_p, ctypes.c_int, ctypes.c_longlong, ctypes.c_double


class ServeTP:
    WAIT_LIMIT_S = 20.0

    def __init__(self, group: Any = None, native: Optional[bool] = None, slot_rows: int = 4096,
                 max_ctas: int = 16, multimem: Optional[bool] = None) -> None:
        self.group = group or dist.group.WORLD
        self.size, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.native = native
        self.slot_rows = slot_rows
        self.max_ctas = max_ctas
        # True: in-switch reduction (required); False: plain peer stores (the push kernel); None: the
        # environment decides - KOTODAMA_SERVE_MULTIMEM=1 uses the in-switch form where the buffers have a
        # multicast mapping.  Off by default: in its one-shot form every rank still reads the whole vector,
        # so the bytes each GPU serves are those of the push form, and it measured 2 % slower at TP 2
        # (p50 7.50 against 7.33 ms per 64-request decode step).
        if multimem is None and os.environ.get("KOTODAMA_SERVE_MULTIMEM", "0") != "1":
            multimem = False
        self.multimem = multimem
        self.fused_gemm = os.environ.get("KOTODAMA_SERVE_FUSED_AR", "1") == "1"   # GEMM + all-reduce in one launch (decode)
        self.fused_calls = 0
        self.native_calls = 0
        self.multimem_calls = 0
        self.library_calls = 0
        self._ready = False

    def prepare_model(self, model: torch.nn.Module) -> None:
        from ..parallel.tp import apply_tensor_parallelism
        if not any(hasattr(p, "_tp_shard_dim") for p in model.parameters()):
            apply_tensor_parallelism(model, self.group)

    # ------------------------------------------------------------------ native all-reduce
    def _setup(self, device: torch.device, width: int, ops: Any) -> None:
        import torch.distributed._symmetric_memory as symm_mem
        from ..ops import _build
        self.lib = _build.load()
        self.ops = ops
        self.slot_elems = self.slot_rows * width
        self.recv = symm_mem.empty(2 * self.size * self.slot_elems, dtype=torch.bfloat16, device=device)
        self.flags = symm_mem.empty(16, dtype=torch.int32, device=device)
        self.flags.zero_()
        h_r = symm_mem.rendezvous(self.recv, self.group)
        h_f = symm_mem.rendezvous(self.flags, self.group)
        self._handles = (h_r, h_f)
        arr = lambda ptrs: (_VP * 8)(*([int(p) for p in ptrs] + [0] * (8 - len(ptrs))))
        self.recv_ptrs, self.flag_ptrs = arr(h_r.buffer_ptrs), arr(h_f.buffer_ptrs)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.counters = torch.zeros(2, dtype=torch.int32, device=device)
        # in-switch reduction: the partial stays in this rank's own symmetric buffer and one
        # multimem.ld_reduce per 16 bytes returns the sum over all ranks (needs a multicast mapping of
        # the buffer, which the symmetric-memory rendezvous provides on NVSwitch systems)
        self.mc_ptr = 0
        if self.multimem is not False:
            self.mm_buf = symm_mem.empty(2 * self.slot_elems, dtype=torch.bfloat16, device=device)
            h_m = symm_mem.rendezvous(self.mm_buf, self.group)
            self._h_m = h_m
            self.mc_ptr = int(getattr(h_m, "multicast_ptr", 0) or 0)
            self.mm_flags = symm_mem.empty(16, dtype=torch.int32, device=device)
            self.mm_flags.zero_()
            h_mf = symm_mem.rendezvous(self.mm_flags, self.group)
            self.mm_flag_ptrs = arr(h_mf.buffer_ptrs)
            self.mm_epoch = torch.zeros(1, dtype=torch.int32, device=device)
            self.mm_counters = torch.zeros(2, dtype=torch.int32, device=device)
            if self.multimem is True and not self.mc_ptr:
                raise RuntimeError("multimem all-reduce requested, but the symmetric buffer has no multicast mapping")
        torch.cuda.synchronize()
        dist.barrier(group=self.group)
        self._ready = True

    def all_reduce(self, ops: Any, y: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        use_native = self.native if self.native is not None else y.is_cuda
        if use_native and y.is_cuda and y.dtype == torch.bfloat16 and y.shape[-1] % 8 == 0:
            if not self._ready:
                self._setup(y.device, y.shape[-1], ops)
            fits = y.numel() <= self.slot_elems and y.is_contiguous() and (residual is None or residual.is_contiguous())
            if fits and self.mc_ptr:
                out = torch.empty_like(y)
                rc = self.lib.kb_allreduce_multimem(
                    _VP(y.data_ptr()), _LL(y.numel()), _LL(self.slot_elems), _VP(self.mm_buf.data_ptr()), _VP(self.mc_ptr),
                    self.mm_flag_ptrs, _I(self.size), _I(self.rank),
                    _VP(residual.data_ptr() if residual is not None else None), _VP(out.data_ptr()),
                    _VP(self.mm_epoch.data_ptr()), _VP(self.mm_counters.data_ptr()), _D(self.WAIT_LIMIT_S),
                    _VP(ops.status(y.device).data_ptr()), _I(self.max_ctas), _VP(torch.cuda.current_stream().cuda_stream))
                ops.launches += 1
                if rc != 0:
                    raise RuntimeError(f"kb_allreduce_multimem: launcher returned {rc}")
                self.native_calls += 1
                self.multimem_calls += 1
                return out
            if fits:
                out = torch.empty_like(y)
                rc = self.lib.kb_allreduce_push(
                    _VP(y.data_ptr()), _LL(y.numel()), _LL(self.slot_elems), self.recv_ptrs, self.flag_ptrs,
                    _I(self.size), _I(self.rank), _VP(residual.data_ptr() if residual is not None else None),
                    _VP(out.data_ptr()), _VP(self.epoch.data_ptr()), _VP(self.counters.data_ptr()),
                    _D(self.WAIT_LIMIT_S), _VP(ops.status(y.device).data_ptr()), _I(self.max_ctas),
                    _VP(torch.cuda.current_stream().cuda_stream))
                ops.launches += 1
                if rc != 0:
                    raise RuntimeError(f"kb_allreduce_push: launcher returned {rc}")
                self.native_calls += 1
                return out
        self.library_calls += 1
        y = y.contiguous()
        dist.all_reduce(y, group=self.group)
        return y if residual is None else y + residual

    def sync_tokens(self, toks: Any, device: torch.device) -> list[int]:
        """Rank 0's sampled tokens for every rank.  Replicated work is not bitwise identical across
        ranks (split-K products add in atomic order), so near-ties could otherwise be broken
        differently and the ranks' request sets would drift apart."""
        t = torch.as_tensor(toks, dtype=torch.int64).to(device)
        dist.broadcast(t, src=dist.get_global_rank(self.group, 0), group=self.group)
        return t.tolist()

    def row_linear(self, ops: Any, x: torch.Tensor, w: Any, residual: Optional[torch.Tensor]) -> torch.Tensor:
        """Row-parallel projection + all-reduce (+ residual).  Decode-size inputs on CUDA take one launch: the
        cluster split-K product whose epilogue pushes the tile rows to every rank and sums all ranks' slots
        (``kb_gemm_skinny_allreduce``); everything else is the product followed by ``all_reduce``."""
        wt = getattr(w, "w", w)
        use_native = self.native if self.native is not None else x.is_cuda
        if (self.fused_gemm and use_native and x.is_cuda and isinstance(wt, torch.Tensor) and x.dtype == torch.bfloat16
                and wt.dtype == torch.bfloat16 and x.dim() == 2 and x.shape[0] <= 128 and wt.shape[0] % 8 == 0
                and wt.shape[1] >= 256 and x.stride(-1) == 1 and x.stride(0) % 8 == 0 and wt.is_contiguous()
                and getattr(ops, "skinny_cluster", False) and not self.mc_ptr_requested()
                and (residual is None or residual.is_contiguous())):
            if not self._ready:
                self._setup(x.device, wt.shape[0], ops)
            M, K = x.shape
            N = wt.shape[0]
            if M * N <= self.slot_elems and not self.mc_ptr:
                out = torch.empty(M, N, device=x.device, dtype=torch.bfloat16)
                packed = getattr(w, "packed", None)
                rc = self.lib.kb_gemm_skinny_allreduce(
                    _VP(x.data_ptr()), _VP((packed if packed is not None else wt).data_ptr()), _VP(out.data_ptr()),
                    _VP(residual.data_ptr() if residual is not None else None), _I(M), _I(N), _I(K), _LL(x.stride(0)),
                    _LL(K), _I(int(packed is not None) | (2 if hasattr(w, "w") else 0)), self.recv_ptrs, self.flag_ptrs, _I(self.size), _I(self.rank),
                    _LL(self.slot_elems), _VP(self.epoch.data_ptr()), _VP(self.counters.data_ptr()), _D(self.WAIT_LIMIT_S),
                    _VP(ops.status(x.device).data_ptr()), _VP(torch.cuda.current_stream().cuda_stream))
                if rc == 0:
                    ops.launches += 1
                    self.native_calls += 1
                    self.fused_calls += 1
                    return out
                if rc != 9:
                    raise RuntimeError(f"kb_gemm_skinny_allreduce: launcher returned {rc}")
                self.fused_gemm = False              # the grid cannot be resident at once on this device: two launches
        return self.all_reduce(ops, ops.gemm_nt(x, w), residual)

    def mc_ptr_requested(self) -> bool:
        return self.multimem is True


# ---------------------------------------------------------------------------- lock-step driving
class _Control:
    """Rank 0 -> followers, once per step: a fixed-size header tensor ``[stop, body bytes, step,
    0]`` on the group's device, followed - only when requests were admitted or cancelled since
    the last step - by a byte tensor with their JSON.  A decode step without admissions costs one
    32-byte broadcast; nothing is pickled."""

    def __init__(self, tp: ServeTP, device: torch.device) -> None:
        self.group = tp.group
        self.src = dist.get_global_rank(tp.group, 0)
        # NCCL moves device tensors, gloo host tensors
        self.device = device if dist.get_backend(tp.group) == "nccl" else torch.device("cpu")
        self.step_no = 0
        self.header_bytes = 0
        self.body_bytes = 0

    def send(self, stop: bool, new: list, cancel: list) -> None:
        body = b""
        if new or cancel:
            body = json.dumps({"new": [[p, dataclasses.asdict(sp) if sp is not None else None] for p, sp in new],
                               "cancel": cancel}).encode()
        self.step_no += 1
        hdr = torch.tensor([int(stop), len(body), self.step_no, 0], dtype=torch.int64).to(self.device)
        dist.broadcast(hdr, src=self.src, group=self.group)
        self.header_bytes += 32
        if body:
            t = torch.frombuffer(bytearray(body), dtype=torch.uint8).to(self.device)
            dist.broadcast(t, src=self.src, group=self.group)
            self.body_bytes += len(body)

    def recv(self) -> tuple[bool, list, list]:
        hdr = torch.zeros(4, dtype=torch.int64, device=self.device)
        dist.broadcast(hdr, src=self.src, group=self.group)
        stop, n, step_no, _ = hdr.tolist()
        self.step_no += 1
        if step_no != self.step_no:
            raise RuntimeError(f"tensor-parallel serving: follower at step {self.step_no}, leader at {step_no}")
        if n == 0:
            return bool(stop), [], []
        t = torch.empty(n, dtype=torch.uint8, device=self.device)
        dist.broadcast(t, src=self.src, group=self.group)
        msg = json.loads(bytes(t.cpu().numpy()))
        from .engine import SamplingParams
        new = [(p, SamplingParams(**sp) if sp is not None else None) for p, sp in msg["new"]]
        return bool(stop), new, msg["cancel"]


class TPLeader:
    """Rank 0's view of a tensor-parallel engine: admissions and cancellations are queued here and
    shipped to the followers at the start of the next step, so every rank applies them at the same
    point of the schedule."""

    def __init__(self, engine: Any, tp: ServeTP) -> None:
        self.engine, self.tp = engine, tp
        self.control = _Control(tp, engine.device)
        self._pending: list = []
        self._cancels: list = []

    def __getattr__(self, name: str) -> Any:        # everything else (cache, stats, ...) is the engine's
        return getattr(self.engine, name)

    def add_request(self, prompt: list[int], params: Any = None):
        r = self.engine.add_request(prompt, params)
        self._pending.append((list(prompt), params))
        return r

    def cancel(self, rid: int) -> bool:
        """Takes effect at the next step boundary on every rank (request ids are assigned in admission
        order, so they agree across ranks)."""
        self._cancels.append(int(rid))
        return True

    def step(self):
        self.control.send(False, self._pending, self._cancels)
        for rid in self._cancels:
            self.engine.cancel(rid)
        self._pending, self._cancels = [], []
        return self.engine.step()

    def has_work(self) -> bool:
        return self.engine.has_work()

    def shutdown(self) -> None:
        self.control.send(True, [], [])

    def generate(self, prompts: list[list[int]], params: Any = None) -> list[list[int]]:
        reqs = [self.add_request(p, params) for p in prompts]
        while self.has_work():
            self.step()
        return [r.generated for r in reqs]


def run_follower(engine: Any, tp: ServeTP) -> list:
    """Loop of the ranks other than 0: mirror the leader's admissions and cancellations, run the
    same steps.  Returns the mirrored requests in admission order."""
    control = _Control(tp, engine.device)
    reqs = []
    while True:
        stop, new, cancel = control.recv()
        if stop:
            return reqs
        for prompt, params in new:
            reqs.append(engine.add_request(prompt, params))
        for rid in cancel:
            engine.cancel(rid)
        engine.step()
