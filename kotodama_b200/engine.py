"""Hand-scheduled training executor.

Instead of tracing the model with autograd (or a compiler) the decoder stack is run by an
explicit forward schedule that records what the backward needs, and an explicit backward
schedule that consumes it.  That gives the executor what a B200 step needs and autograd
cannot express:

* all parameters, gradients and optimizer state live in flat arenas (one allocation each,
  peer-mappable), ``q/k/v`` and ``gate/up`` are adjacent so one GEMM serves each group while
  the checkpoint still sees the reference's separate tensors;
* AttnRes source gradients are accumulated *in place* by the routing-backward kernel (no
  per-call gradient tensors, no re-stacking of sources: the sources are passed by pointer);
* a layer's gradients are final as soon as its backward is done, so the gradient
  reduction of layer ``i`` is launched on the communication stream while layer ``i-1`` is
  still in backward, and Muon work is owner-computes.

Semantics follow the reference loop ``src/training/train.py:567-657`` (micro-steps, loss/GA,
global-norm clip before both optimizers, Muon then AdamW) and the model
``src/model/llama.py:666-716``.  Every op goes through an ops backend
(``kotodama_b200.ops``): PyTorch on CPU, sm_100a kernels on CUDA.
"""
from __future__ import annotations

import os

import math
from dataclasses import dataclass, field
from typing import Any, Optional

import torch
import torch.nn as nn

from .config import ModelConfig
from .models.llama import KotodamaModel
from .optim.muon import resolve_ns_coefficients
from .ops import get_ops
from .ops.reference import Fp8Weight

_ALIGN = 64  # elements; keeps every tensor 128-byte aligned in bf16


def _round_up(x: int, a: int) -> int:
    return (x + a - 1) // a * a


@dataclass
class _Slot:
    name: str
    param: nn.Parameter
    offset: int
    numel: int
    shape: tuple
    kind: str                      # "muon" | "adamw"
    layer: int = -1
    owner: int = 0                 # rank that runs Newton-Schulz for this matrix


class ParamArena:
    """Flat parameter/gradient storage with the model's parameters re-pointed into it.

    Layout: per layer ``[q|k|v] [o] [gate|up] [down]`` (the Muon region), then the embedding,
    then every 1-D parameter in ``named_parameters`` order (the AdamW region).  The Muon rule is
    the reference's: 2-D and neither "embed" nor "lm_head" in the name (``muon.py:381``).
    """

    def __init__(self, model: KotodamaModel, device: torch.device, dtype: torch.dtype,
                 allocator=None, with_grads: bool = True) -> None:
        self.model = model
        named = [(n, p) for n, p in model.named_parameters() if p.requires_grad]
        self.names = [n for n, _ in named]
        muon, adamw = [], []
        for n, p in named:
            (muon if (p.ndim == 2 and "embed" not in n and "lm_head" not in n) else adamw).append((n, p))
        # Muon region in layer order with the fused groups adjacent.
        order_in_layer = ["attn.q_proj", "attn.k_proj", "attn.v_proj", "attn.o_proj",
                          "ffn.gate_proj", "ffn.up_proj", "ffn.down_proj"]

        def key(item):
            n = item[0]
            parts = n.split(".")
            li = int(parts[1]) if parts[0] == "layers" else 10 ** 6
            sub = ".".join(parts[2:4]) if parts[0] == "layers" else n
            return (li, order_in_layer.index(sub) if sub in order_in_layer else 99)

        muon.sort(key=key)
        self.slots: list[_Slot] = []
        off = 0
        for n, p in muon:
            parts = n.split(".")
            li = int(parts[1]) if parts[0] == "layers" else -1
            fused_follow = any(s in n for s in ("k_proj", "v_proj", "up_proj"))
            if not fused_follow:
                off = _round_up(off, _ALIGN)
            self.slots.append(_Slot(n, p, off, p.numel(), tuple(p.shape), "muon", li))
            off += p.numel()
        self.muon_end = off = _round_up(off, _ALIGN)
        for n, p in adamw:
            off = _round_up(off, _ALIGN)
            self.slots.append(_Slot(n, p, off, p.numel(), tuple(p.shape), "adamw"))
            off += p.numel()
        self.total = _round_up(off, _ALIGN)
        alloc = allocator or (lambda n: torch.zeros(n, device=device, dtype=dtype))
        self.params = alloc(self.total)
        self.grads = alloc(self.total) if with_grads else None
        self.by_name = {s.name: s for s in self.slots}
        owners = {}
        for mod_name, mod in model.named_modules():
            for pn in mod._parameters:
                owners[(mod_name + "." if mod_name else "") + pn] = (mod, pn)
        with torch.no_grad():
            for s in self.slots:
                view = self.params[s.offset:s.offset + s.numel].view(s.shape)
                if not s.param.is_meta:
                    view.copy_(s.param.data)
                mod, pn = owners[s.name]
                newp = nn.Parameter(view, requires_grad=with_grads)
                if with_grads:
                    newp.grad = self.grads[s.offset:s.offset + s.numel].view(s.shape)
                for k, v in vars(s.param).items():          # keep tags such as the tensor-parallel shard info
                    if k.startswith("_tp_"):
                        setattr(newp, k, v)
                mod._parameters[pn] = newp
                s.param = newp
        model.materialize_buffers(device)

    @torch.no_grad()
    def init_weights(self, num_layers: int, seed: int) -> None:
        """Reference initialisation (``llama.py:583-598``) written straight into the arena."""
        gen = torch.Generator(device=self.params.device).manual_seed(seed)
        scale = 1.0 / math.sqrt(2 * num_layers)
        for s in self.slots:
            v = self.params[s.offset:s.offset + s.numel].view(s.shape)
            if len(s.shape) == 2:
                std = 0.02 * (scale if ("o_proj" in s.name or "down_proj" in s.name) else 1.0)
                v.copy_(torch.randn(s.shape, device=v.device, generator=gen) * std)
            elif "query" in s.name:
                v.zero_()
            else:
                v.fill_(1.0)

    def view(self, name: str, grads: bool = False) -> torch.Tensor:
        s = self.by_name[name]
        base = self.grads if grads else self.params
        return base[s.offset:s.offset + s.numel].view(s.shape)

    def fused(self, first: str, last: str, grads: bool = False) -> torch.Tensor:
        """View spanning the adjacent tensors ``first..last`` as one ``[rows, in]`` matrix."""
        a, b = self.by_name[first], self.by_name[last]
        base = self.grads if grads else self.params
        cols = a.shape[1]
        return base[a.offset:b.offset + b.numel].view(-1, cols)

    def muon_slots(self) -> list[_Slot]:
        return [s for s in self.slots if s.kind == "muon"]

    def adamw_range(self) -> tuple[int, int]:
        return self.muon_end, self.total


@dataclass
class _LayerRec:
    srcs1: list = field(default_factory=list)
    stats1: Any = None
    xn1: Any = None
    qkv: Any = None
    qk: Any = None
    rstd_qk: Any = None
    attn_o: Any = None
    lse: Any = None
    part_after_attn: Any = None
    srcs2: list = field(default_factory=list)
    stats2: Any = None
    xn2: Any = None
    gu: Any = None
    act: Any = None
    part_before_attn: Any = None   # None when the attention output starts a new block
    part_after_mlp: Any = None


class _OptView:
    """What the LR scheduler and the checkpoint manager need from an optimizer: ``defaults``,
    ``param_groups`` and the torch-layout ``state_dict`` / ``load_state_dict``."""

    def __init__(self, lr: float, state_fn=None, load_fn=None, **hyper: Any) -> None:
        self.defaults = dict(lr=lr, **hyper)
        self.param_groups = [dict(lr=lr, **hyper)]
        self._state_fn, self._load_fn = state_fn, load_fn

    def state_dict(self) -> dict[str, Any]:
        return self._state_fn() if self._state_fn else {}

    def load_state_dict(self, sd: dict[str, Any]) -> None:
        if self._load_fn:
            self._load_fn(sd)

    def zero_grad(self, set_to_none: bool = False) -> None:
        return None


class TrainEngine:
    """Owns arenas, optimizer state and the fwd/bwd/optimizer schedule for one rank."""

    def __init__(self, model: KotodamaModel, *, device: torch.device | str = "cpu",
                 dtype: torch.dtype = torch.float32, comm=None, ops=None,
                 muon_lr: float = 0.03, muon_momentum: float = 0.95, muon_weight_decay: float = 0.01,
                 muon_ns_iterations: int = 5, muon_ns_coefficients: Optional[str] = None,
                 adamw_lr: float = 6e-4, adamw_betas: tuple[float, float] = (0.9, 0.95),
                 adamw_weight_decay: float = 0.1, adamw_eps: float = 1e-8, gradient_clip: float = 1.0,
                 adamw_only: bool = False, ce_chunk: int = 4096, fp8: bool = False,
                 fp8_recipe: str = "block128") -> None:
        from .parallel.comm import LocalComm

        self.device = torch.device(device)
        self.dtype = dtype
        self.model = model
        self.cfg: ModelConfig = model.config
        self.comm = comm or LocalComm()
        self.ops = ops or get_ops(self.device)
        if hasattr(self.comm, "prepare_model"):
            self.comm.prepare_model(model)          # tensor parallelism shards the projections first
        self.arena = ParamArena(model, self.device, dtype, allocator=self.comm.allocator(self.device, dtype))
        self.comm.attach(self)
        self.gradient_clip = gradient_clip
        self.adamw_only = adamw_only
        self.ce_chunk = ce_chunk
        self.fp8, self.fp8_recipe = fp8, fp8_recipe
        self.ns_coefficients = muon_ns_coefficients
        self.ns_batch = 14                 # same-shape matrices per batched Newton-Schulz product
        self.muon_opt = _OptView(muon_lr, self.muon_state_dict, self.load_muon_state_dict, momentum=muon_momentum, nesterov=True,
                                 weight_decay=muon_weight_decay, ns_iterations=muon_ns_iterations)
        self.adamw_opt = _OptView(adamw_lr, self.adamw_state_dict, self.load_adamw_state_dict, betas=tuple(adamw_betas), eps=adamw_eps,
                                  weight_decay=adamw_weight_decay)
        resolve_ns_coefficients(muon_ns_coefficients, muon_ns_iterations)
        # optimizer state
        self.opt_step = 0
        self._assign_owners()
        a0, a1 = self.arena.adamw_range()
        lo = 0 if adamw_only else a0
        self.adamw_lo = lo
        self.exp_avg = torch.zeros(a1 - lo, device=self.device, dtype=torch.float32)
        self.exp_avg_sq = torch.zeros(a1 - lo, device=self.device, dtype=torch.float32)
        self.momentum: dict[str, torch.Tensor] = {}
        if not adamw_only:
            for s in self.arena.muon_slots():
                if s.owner == self.comm.rank or not self.comm.distributed_muon:
                    self.momentum[s.name] = torch.zeros(s.shape, device=self.device, dtype=dtype)
        self._wcache: dict[str, torch.Tensor] = {}
        self._gather_weights()
        self.refresh_fp8()
        # AttnRes routing in blocked form for every block with at least this many committed sources
        self.route_block_min = int(os.environ.get("KOTODAMA_ROUTE_BLOCK_MIN", "2"))
        self._route_plan, self._route_groups = self._make_route_plan()

    @classmethod
    def from_meta(cls, model: KotodamaModel, cfg: ModelConfig, *, seed: int = 0, **kw: Any) -> "TrainEngine":
        """Build from a model whose parameters are on the meta device: weights are initialised on
        the target device directly in the arena (no host copy of a multi-billion-parameter model)."""
        eng = cls(model, **kw)
        eng.arena.init_weights(cfg.num_layers, seed)
        eng.comm.attach(eng)   # re-broadcast: ranks must start from identical weights
        eng.refresh_fp8()
        return eng

    # ------------------------------------------------------------ helpers
    def _assign_owners(self) -> None:
        """Greedy balance of Newton-Schulz FLOPs over ranks (largest first)."""
        world = self.comm.world
        load = [0.0] * world
        slots = self.arena.muon_slots()
        def ns_flops(s):
            r, c = min(s.shape), max(s.shape)
            return 2.0 * r * r * c * 2 + 2.0 * r * r * r
        for s in sorted(slots, key=lambda s: (-ns_flops(s), s.offset)):
            o = min(range(world), key=lambda r: (load[r], r))
            s.owner = o
            load[o] += ns_flops(s)

    def _gather_weights(self) -> None:
        m, ar = self.model, self.arena
        # fp8: the four projections of every layer run in block-scaled e4m3 (forward, data gradient and
        # weight gradient); masters, gradients, optimizer and everything else stay bf16/fp32
        wrap = (lambda t: Fp8Weight(t)) if self.fp8 else (lambda t: t)
        self.layer_w = []
        for i in range(self.cfg.num_layers):
            p = f"layers.{i}."
            self.layer_w.append(dict(
                wqkv=wrap(ar.fused(p + "attn.q_proj.weight", p + "attn.v_proj.weight")),
                wo=wrap(ar.view(p + "attn.o_proj.weight")),
                wgu=wrap(ar.fused(p + "ffn.gate_proj.weight", p + "ffn.up_proj.weight")),
                wd=wrap(ar.view(p + "ffn.down_proj.weight")),
                g_wqkv=ar.fused(p + "attn.q_proj.weight", p + "attn.v_proj.weight", grads=True),
                g_wo=ar.view(p + "attn.o_proj.weight", grads=True),
                g_wgu=ar.fused(p + "ffn.gate_proj.weight", p + "ffn.up_proj.weight", grads=True),
                g_wd=ar.view(p + "ffn.down_proj.weight", grads=True),
            ))

    def refresh_fp8(self) -> None:
        """Re-quantise the projection weights from their bf16 masters (after every optimizer step and
        after a checkpoint load)."""
        if not self.fp8:
            return
        for lw in self.layer_w:
            for k in ("wqkv", "wo", "wgu", "wd"):
                w = lw[k]
                if all(d % 128 == 0 for d in w.shape):
                    w.refresh(self.ops)

    def _p(self, name: str) -> torch.Tensor:
        return self.arena.view(name)

    def _g(self, name: str) -> torch.Tensor:
        return self.arena.view(name, grads=True)

    def _acc_small(self, name: str, val: Optional[torch.Tensor]) -> None:
        if val is None:
            return
        g = self._g(name)
        if self._first_micro:
            g.copy_(val.view(g.shape))
        else:
            g.add_(val.view(g.shape).to(g.dtype))

    # ------------------------------------------------------------ AttnRes routing schedule
    def _route_names(self, j: int) -> tuple[str, str, str]:
        """Parameter names (pseudo-query, key-norm weight, following RMSNorm weight) of routing call
        ``j``: ``2i`` before the attention of layer ``i``, ``2i + 1`` before its MLP, ``2L`` at the output."""
        if j == 2 * self.cfg.num_layers:
            return "final_res_query", "final_res_norm.weight", "norm.weight"
        p = f"layers.{j // 2}."
        if j % 2 == 0:
            return p + "attn_res_query", p + "attn_res_norm.weight", p + "attn_norm.weight"
        return p + "mlp_res_query", p + "mlp_res_norm.weight", p + "ffn_norm.weight"

    def _make_route_plan(self):
        """Groups the routing calls by the set of committed sources they see.  A group starts at the
        pre-attention call of a boundary layer (which sees the finished block as its last source,
        i.e. exactly the committed set of the calls that follow) and runs to the call before the next
        boundary.  Groups with at least ``route_block_min`` committed sources run in blocked form: one
        phase-1 pass for all their queries, then one phase-2 merge per call
        (reference: serve.py:113-164)."""
        cfg = self.cfg
        plan: dict[int, tuple[int, int]] = {}
        groups: list[dict] = []
        if not cfg.attn_res or self.route_block_min <= 0:
            return plan, groups
        bset = self.model._attn_res_boundary_set
        committed, cur = 0, None
        for j in range(2 * cfg.num_layers + 1):
            if j % 2 == 0 and j // 2 in bset and j < 2 * cfg.num_layers:
                committed += 1
                cur = None
                if committed >= self.route_block_min and self.ops.route_blocked_ok(committed, cfg.hidden_size):
                    cur = dict(S=committed, members=[])
                    groups.append(cur)
            if cur is not None:
                plan[j] = (len(groups) - 1, len(cur["members"]))
                cur["members"].append(j)
        return plan, groups

    def _route_fwd(self, j: int, srcs: list, fw: dict):
        """Routing call ``j`` over ``srcs`` (committed sources, then the partial sum) fused with the
        RMSNorm that follows.  Returns the normalised activations and what the backward needs."""
        ops, eps = self.ops, self.cfg.norm_eps
        qn, rn, nn_ = self._route_names(j)
        attn_res = self.cfg.attn_res
        q = self._p(qn) if attn_res else None
        rnw = self._p(rn) if attn_res else None
        ent = self._route_plan.get(j)
        if ent is None:
            xn, stats = ops.route_norm_fwd(srcs, q, rnw, self._p(nn_), eps)
            return xn, ("plain", stats)
        gid, k = ent
        grp = self._route_groups[gid]
        if k == 0:
            assert len(srcs) == grp["S"]
            names = [self._route_names(m) for m in grp["members"]]
            qs = torch.stack([self._p(n[0]) for n in names])
            rns = torch.stack([self._p(n[1]) for n in names])
            o, lse, st = ops.route_p1_fwd(srcs, qs, rns, eps)
            fw[gid] = dict(o=o, lse=lse, stats=st, srcs=list(srcs), qs=qs, rns=rns, dw2={})
            partial = None
        else:
            assert len(srcs) == grp["S"] + 1
            partial = srcs[-1]
        g = fw[gid]
        xn, st2 = ops.route_p2_fwd(g["o"][k], g["lse"][k], partial, q, rnw, self._p(nn_), eps)
        return xn, ("blocked", gid, k, partial, st2)

    def _route_bwd(self, j: int, dxn: torch.Tensor, srcs: list, saved, fw: dict, dsrc_list) -> None:
        """Backward of :meth:`_route_fwd`: source gradients are written or accumulated in place,
        parameter gradients go to the arena."""
        ops, eps = self.ops, self.cfg.norm_eps
        qn, rn, nn_ = self._route_names(j)
        attn_res = self.cfg.attn_res
        q = self._p(qn) if attn_res else None
        rnw = self._p(rn) if attn_res else None
        if saved[0] == "plain":
            ds, acc = dsrc_list(srcs)
            dq, drn, dnw = ops.route_norm_bwd(dxn, srcs, q, rnw, self._p(nn_), eps, saved[1], ds, acc)
            self._acc_small(nn_, dnw)
            if attn_res:
                self._acc_small(qn, dq)
                self._acc_small(rn, drn)
            return
        _, gid, k, partial, st2 = saved
        g = fw[gid]
        if "do" not in g:
            g["do"] = torch.empty_like(g["o"])
            g["dlse"] = torch.empty_like(g["lse"])
        dpart, pacc = None, False
        if partial is not None:
            (dpart,), (pacc,) = dsrc_list([partial])
        dw2, dnw = ops.route_p2_bwd(dxn, g["o"][k], g["lse"][k], partial, q, rnw, self._p(nn_), eps, st2,
                                    g["do"][k], g["dlse"][k], dpart, pacc)
        self._acc_small(nn_, dnw)
        g["dw2"][k] = dw2
        if k != 0:
            return
        ds, acc = dsrc_list(g["srcs"])
        dws = ops.route_p1_bwd(g["srcs"], g["qs"], g["rns"], g["do"], g["dlse"], g["lse"], g["stats"], ds, acc)
        for mk, m in enumerate(self._route_groups[gid]["members"]):
            dw = dws[mk] if g["dw2"].get(mk) is None else dws[mk] + g["dw2"][mk]
            mq, mr, _ = self._route_names(m)
            self._acc_small(mq, dw * self._p(mr).float())
            self._acc_small(mr, dw * self._p(mq).float())
        fw.pop(gid)

    # ------------------------------------------------------------ forward
    @torch.no_grad()
    def forward_backward(self, input_ids: torch.Tensor, loss_scale: float = 1.0, first_micro: bool = True,
                         last_micro: bool = True, need_grad: bool = True):
        """One micro-batch ``input_ids[B,T]``: returns ``(loss, z_loss)`` as 0-dim device tensors
        (``loss`` includes the z-loss) and leaves gradients of ``loss_scale * loss`` in the arena
        (overwritten on the first micro-step, accumulated afterwards)."""
        ops, cfg, ar = self.ops, self.cfg, self.arena
        self._first_micro = first_micro
        B, T = input_ids.shape
        N = B * T
        H, KV, hd, D, F_ = cfg.num_attention_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
        if self.comm.tp_size > 1:
            H, KV, F_ = H // self.comm.tp_size, KV // self.comm.tp_size, F_ // self.comm.tp_size
        eps = cfg.norm_eps
        labels = torch.roll(input_ids, -1, dims=1)
        labels[:, -1] = -100
        ids = self.comm.shard_tokens(input_ids.reshape(-1))          # sequence parallelism: this rank's tokens
        labels = self.comm.shard_tokens(labels.reshape(-1))
        n_valid = self.comm.loss_reduce((labels >= 0).sum().float().reshape(1)).clamp(min=1)
        wemb = self._p("embed_tokens.weight")
        cos, sin = self.model.rope_cos, self.model.rope_sin
        attn_res = cfg.attn_res
        bset = self.model._attn_res_boundary_set if attn_res else frozenset()
        fw: dict = {}                                               # blocked routing groups in flight

        embed = ops.embedding_fwd(ids, wemb)
        committed: list[torch.Tensor] = []
        partial: Optional[torch.Tensor] = embed
        recs: list[_LayerRec] = []
        for i in range(cfg.num_layers):
            lw = self.layer_w[i]
            p = f"layers.{i}."
            r = _LayerRec()
            r.srcs1 = committed + [partial]
            r.xn1, r.stats1 = self._route_fwd(2 * i, r.srcs1, fw)
            if i in bset:
                committed = committed + [partial]
                partial = None
            r.part_before_attn = partial
            r.qkv = self.comm.col_linear(ops, r.xn1, lw["wqkv"])
            r.qk, r.rstd_qk = ops.qknorm_rope_fwd(
                r.qkv, self._p(p + "attn.q_norm.weight") if cfg.qk_norm else None,
                self._p(p + "attn.k_norm.weight") if cfg.qk_norm else None, cos, sin, T, H, KV, hd, eps)
            Nq = r.qkv.shape[0]
            q4 = r.qk[:, : H * hd].view(Nq // T, T, H, hd)
            k4 = r.qk[:, H * hd:].view(Nq // T, T, KV, hd)
            v4 = r.qkv[:, (H + KV) * hd:].view(Nq // T, T, KV, hd)
            r.attn_o, r.lse = ops.attention_fwd(q4, k4, v4)
            partial = self.comm.row_linear(ops, r.attn_o.view(Nq, H * hd), lw["wo"], residual=partial)
            r.part_after_attn = partial
            r.srcs2 = committed + [partial]
            r.xn2, r.stats2 = self._route_fwd(2 * i + 1, r.srcs2, fw)
            r.gu = self.comm.col_linear(ops, r.xn2, lw["wgu"])
            r.act = ops.swiglu_fwd(r.gu)
            partial = self.comm.row_linear(ops, r.act, lw["wd"], residual=partial)
            r.part_after_mlp = partial
            if not need_grad:
                r = _LayerRec()
            recs.append(r)
        fsrcs = committed + [partial]
        xf, fstats = self._route_fwd(2 * cfg.num_layers, fsrcs, fw)
        wl = self.model.get_lm_head_weight()
        g_wl = self._g("embed_tokens.weight") if self.model.lm_head is None else self._g("lm_head.weight")
        ce, zl, dxf = ops.linear_ce(xf, wl, labels, cfg.z_loss_weight, loss_scale,
                                    g_wl if need_grad else None, dw_accumulate=not first_micro,
                                    chunk=self.ce_chunk, need_grad=need_grad, count=n_valid)
        if self.comm.tp_size > 1:
            both = self.comm.loss_reduce(torch.stack([ce.reshape(()), zl.reshape(())]).float())
            ce, zl = both[0], both[1]
        loss = ce + zl
        if not need_grad:
            return loss, zl
        if self.model.lm_head is not None and first_micro:
            self._g("embed_tokens.weight").zero_()

        # ---------------------------------------------------------- backward
        grads: dict[int, torch.Tensor] = {}

        def dsrc_list(srcs):
            out, acc = [], []
            for s in srcs:
                k = id(s)
                if k in grads:
                    out.append(grads[k]); acc.append(True)
                else:
                    g = torch.empty_like(s)
                    grads[k] = g
                    out.append(g); acc.append(False)
            return out, acc

        self._route_bwd(2 * cfg.num_layers, dxf, fsrcs, fstats, fw, dsrc_list)
        del dxf, xf
        for i in reversed(range(cfg.num_layers)):
            lw, r, p = self.layer_w[i], recs[i], f"layers.{i}."
            # ---- MLP sub-layer
            dP = grads[id(r.part_after_mlp)]
            dact = self.comm.row_linear_bwd(ops, dP, lw["wd"], r.act, lw["g_wd"], not first_micro)
            dgu = ops.swiglu_bwd(r.gu, dact)
            del dact
            dxn2 = self.comm.col_linear_bwd(ops, dgu, lw["wgu"], r.xn2, lw["g_wgu"], not first_micro)
            del dgu
            grads[id(r.part_after_attn)] = dP                      # residual add: gradient passes through
            self._route_bwd(2 * i + 1, dxn2, r.srcs2, r.stats2, fw, dsrc_list)
            del dxn2
            # ---- attention sub-layer
            dP = grads[id(r.part_after_attn)]
            Nq = r.qkv.shape[0]
            dattn = self.comm.row_linear_bwd(ops, dP, lw["wo"], r.attn_o.view(Nq, H * hd), lw["g_wo"], not first_micro)
            dqkv = torch.empty_like(r.qkv)
            dqk = torch.empty_like(r.qk)
            q4 = r.qk[:, : H * hd].view(Nq // T, T, H, hd)
            k4 = r.qk[:, H * hd:].view(Nq // T, T, KV, hd)
            v4 = r.qkv[:, (H + KV) * hd:].view(Nq // T, T, KV, hd)
            ops.attention_bwd(dattn.view(Nq // T, T, H, hd), q4, k4, v4, r.attn_o, r.lse,
                              dqk[:, : H * hd].view(Nq // T, T, H, hd), dqk[:, H * hd:].view(Nq // T, T, KV, hd),
                              dqkv[:, (H + KV) * hd:].view(Nq // T, T, KV, hd))
            del dattn
            dqw, dkw = ops.qknorm_rope_bwd(
                dqk, r.qkv, self._p(p + "attn.q_norm.weight") if cfg.qk_norm else None,
                self._p(p + "attn.k_norm.weight") if cfg.qk_norm else None, cos, sin, r.rstd_qk, T, H, KV, hd, dqkv)
            if cfg.qk_norm:
                self._acc_small(p + "attn.q_norm.weight", dqw)
                self._acc_small(p + "attn.k_norm.weight", dkw)
            del dqk
            dxn1 = self.comm.col_linear_bwd(ops, dqkv, lw["wqkv"], r.xn1, lw["g_wqkv"], not first_micro)
            del dqkv
            if r.part_before_attn is not None:
                grads[id(r.part_before_attn)] = dP
            self._route_bwd(2 * i, dxn1, r.srcs1, r.stats1, fw, dsrc_list)
            del dxn1
            recs[i] = None  # free activations of this layer
            if last_micro:
                self.comm.layer_grads_ready(i)
        ops.embedding_bwd(grads[id(embed)], ids, self._g("embed_tokens.weight"))
        if last_micro:
            self.comm.small_grads_ready()
        return loss, zl

    # ---------------------------------------------------------- optimizer
    @torch.no_grad()
    def optimizer_step(self) -> torch.Tensor:
        """Clip by global norm, Muon on matrices (owner-computes when distributed), AdamW on the
        rest.  Returns the pre-clip gradient norm (0-dim device tensor)."""
        ops, ar, comm = self.ops, self.arena, self.comm
        comm.finish_grad_reduce()
        total_sq = comm.grad_sumsq(ops)
        norm = total_sq.sqrt()
        if self.gradient_clip > 0:
            coef = (self.gradient_clip / (norm + 1e-6)).clamp(max=1.0)
        else:
            coef = torch.ones((), device=self.device, dtype=torch.float32)
        self.opt_step += 1
        if not self.adamw_only:
            g = self.muon_opt.param_groups[0]
            coeffs = resolve_ns_coefficients(self.ns_coefficients, g["ns_iterations"])
            owned = [s for s in ar.muon_slots() if not (comm.distributed_muon and s.owner != comm.rank)]
            if comm.tp_size == 1:
                # Same-shape matrices are orthogonalised as one batched product: a single 3072x3072
                # Gram matrix is 78 upper-triangle tiles for 74 CTA pairs (two waves, the second almost
                # empty), a batch fills the waves.  Memory is bounded by ``ns_batch`` matrices at a time.
                prepared = []
                for s in owned:
                    grad = ar.view(s.name, grads=True)
                    x, sq = ops.muon_momentum(grad, self.momentum[s.name], g["momentum"], g["nesterov"], coef)
                    rows, cols = s.shape
                    transposed = rows > cols
                    if transposed:
                        x = ops.transpose(x)
                    prepared.append([s, ops.ns_normalize(x, sq), transposed, rows, cols])
                groups: dict[tuple, list] = {}
                for it in prepared:
                    groups.setdefault(tuple(it[1].shape), []).append(it)
                for items in groups.values():
                    for c0 in range(0, len(items), self.ns_batch):
                        chunk = items[c0:c0 + self.ns_batch]
                        xb = torch.stack([it[1] for it in chunk]) if len(chunk) > 1 else chunk[0][1]
                        for (a, b, c) in coeffs:
                            xb = ops.ns_iteration(xb, a, b, c)
                        for i, it in enumerate(chunk):
                            it[1] = xb[i] if len(chunk) > 1 else xb
                for s, x, transposed, rows, cols in prepared:
                    comm.muon_apply(ops, s, x, g["lr"], g["weight_decay"], max(1.0, (rows / cols) ** 0.5), transposed)
                owned = []
            if comm.tp_size > 1 and hasattr(comm, "muon_exchange_group"):
                # Tensor parallelism: matrices of one shape and shard dimension travel together.  Two
                # all-to-alls per group bring whole matrices to their owners and the results back, and
                # every owner orthogonalises its share as one batch.
                tgroups: dict[tuple, list] = {}
                for s in owned:
                    tgroups.setdefault((tuple(comm.full_shape(s)), tuple(s.shape)), []).append(s)
                for (full_shape, _), slots in tgroups.items():
                    rows, cols = full_shape
                    transposed = rows > cols
                    shards = [ops.muon_momentum(ar.view(s.name, grads=True), self.momentum[s.name], g["momentum"],
                                                g["nesterov"], coef)[0] for s in slots]

                    def orthogonalise(batch: torch.Tensor) -> torch.Tensor:
                        xs = []
                        for m in batch:                          # per-matrix Frobenius normalisation
                            xm = ops.transpose(m) if transposed else m
                            xs.append(ops.ns_normalize(xm, ops.sumsq(m)))
                        out = []
                        for c0 in range(0, len(xs), self.ns_batch):
                            chunk = xs[c0:c0 + self.ns_batch]
                            xb = torch.stack(chunk) if len(chunk) > 1 else chunk[0]
                            for (a, b, c) in coeffs:
                                xb = ops.ns_iteration(xb, a, b, c)
                            out += list(xb) if len(chunk) > 1 else [xb]
                        # back to the parameter's orientation and dtype
                        return torch.stack([(ops.transpose(o) if transposed else o).to(batch.dtype) for o in out])

                    res = comm.muon_exchange_group(slots, shards, orthogonalise)
                    scale = max(1.0, (rows / cols) ** 0.5)
                    for s, x in zip(slots, res):
                        comm.muon_apply(ops, s, x.contiguous(), g["lr"], g["weight_decay"], scale, False)
                owned = []
            for s in owned:
                grad = ar.view(s.name, grads=True)
                x, sq = ops.muon_momentum(grad, self.momentum[s.name], g["momentum"], g["nesterov"], coef)
                rows, cols = comm.full_shape(s)
                transposed = rows > cols
                x = comm.muon_gather(s, x)
                if comm.runs_ns(s):                       # under TP one rank orthogonalises the gathered matrix
                    if comm.tp_size > 1:
                        sq = ops.sumsq(x)
                    if transposed:
                        x = ops.transpose(x)
                    x = ops.ns_normalize(x, sq)
                    for (a, b, c) in coeffs:
                        x = ops.ns_iteration(x, a, b, c)
                x = comm.muon_scatter(s, x, transposed)
                if comm.tp_size > 1:
                    transposed = False                    # shards come back in the parameter's orientation
                scale = max(1.0, (rows / cols) ** 0.5)
                comm.muon_apply(ops, s, x, g["lr"], g["weight_decay"], scale, transposed)
        ga = self.adamw_opt.param_groups[0]
        lo, hi = self.adamw_lo, ar.total
        ops.adamw_step(ar.params[lo:hi], ar.grads[lo:hi], self.exp_avg, self.exp_avg_sq, self.opt_step,
                       ga["lr"], ga["betas"][0], ga["betas"][1], ga["eps"], ga["weight_decay"], coef)
        comm.finish_param_publish()
        self.refresh_fp8()
        return norm

    def train_step(self, micro_batches: list[torch.Tensor], keep_grads: bool = True) -> dict[str, torch.Tensor]:
        """One optimizer step over ``len(micro_batches)`` micro-batches (host tensors are copied
        to the device asynchronously).  Returns device scalars ``loss``, ``z_loss``, ``grad_norm``."""
        ga = len(micro_batches)
        loss_acc = zl_acc = None
        for j, mb in enumerate(micro_batches):
            mb = mb.to(self.device, non_blocking=True)
            loss, zl = self.forward_backward(mb, 1.0 / (ga * self.comm.dp_size), j == 0, j == ga - 1)
            loss_acc = loss if loss_acc is None else loss_acc + loss
            zl_acc = zl if zl_acc is None else zl_acc + zl
        norm = self.optimizer_step()
        return {"loss": loss_acc / ga, "z_loss": zl_acc / ga, "grad_norm": norm}

    def after_load(self) -> None:
        """Hook after a checkpoint was copied into the arena (derived copies are refreshed here)."""
        self.comm.attach(self)
        self.refresh_fp8()

    def check(self) -> None:
        """Raise if a kernel reported a timed-out wait."""
        if hasattr(self.ops, "check_status"):
            self.ops.check_status()

    @torch.no_grad()
    def eval_loss(self, input_ids: torch.Tensor) -> torch.Tensor:
        return self.forward_backward(input_ids.to(self.device), need_grad=False)[0]

    # ------------------------------------------------------- checkpoint IO
    def muon_state_dict(self) -> dict[str, Any]:
        """torch-optimizer layout with one ``momentum_buffer`` per Muon parameter in
        ``named_parameters`` order, plus ``ns_coefficients`` (``muon.py:231-234``)."""
        if self.adamw_only:
            return {}
        names = [n for n in self.arena.names if self.arena.by_name[n].kind == "muon"]
        state = {}
        for i, n in enumerate(names):
            buf = self.comm.gather_momentum(self.arena.by_name[n], self.momentum.get(n))
            if buf is not None and self.opt_step > 0:
                state[i] = {"momentum_buffer": buf.detach().cpu().clone()}
        g = dict(self.muon_opt.param_groups[0])
        g["params"] = list(range(len(names)))
        return {"state": state, "param_groups": [g], "ns_coefficients": self.ns_coefficients}

    def load_muon_state_dict(self, sd: dict[str, Any]) -> None:
        if not sd or self.adamw_only:
            return
        names = [n for n in self.arena.names if self.arena.by_name[n].kind == "muon"]
        if sd.get("ns_coefficients") is not None:
            self.ns_coefficients = sd["ns_coefficients"]
        for i, n in enumerate(names):
            st = sd.get("state", {}).get(i)
            if st is not None and n in self.momentum:
                self.momentum[n].copy_(self.comm.shard_like(self.arena.by_name[n], st["momentum_buffer"]))
        if sd.get("param_groups"):
            for k in ("lr", "momentum", "weight_decay", "ns_iterations", "nesterov"):
                if k in sd["param_groups"][0]:
                    self.muon_opt.param_groups[0][k] = sd["param_groups"][0][k]

    def adamw_state_dict(self) -> dict[str, Any]:
        names = [n for n in self.arena.names if self.adamw_only or self.arena.by_name[n].kind == "adamw"]
        state = {}
        if self.opt_step > 0:
            for i, n in enumerate(names):
                s = self.arena.by_name[n]
                o = s.offset - self.adamw_lo
                state[i] = {"step": torch.tensor(float(self.opt_step)),
                            "exp_avg": self.exp_avg[o:o + s.numel].view(s.shape).cpu().clone(),
                            "exp_avg_sq": self.exp_avg_sq[o:o + s.numel].view(s.shape).cpu().clone()}
        g = dict(self.adamw_opt.param_groups[0])
        g.update(amsgrad=False, maximize=False, foreach=None, capturable=False, differentiable=False,
                 fused=None, params=list(range(len(names))))
        return {"state": state, "param_groups": [g]}

    def load_adamw_state_dict(self, sd: dict[str, Any]) -> None:
        if not sd:
            return
        names = [n for n in self.arena.names if self.adamw_only or self.arena.by_name[n].kind == "adamw"]
        for i, n in enumerate(names):
            st = sd.get("state", {}).get(i)
            if st is None:
                continue
            s = self.arena.by_name[n]
            o = s.offset - self.adamw_lo
            self.exp_avg[o:o + s.numel].copy_(st["exp_avg"].reshape(-1))
            self.exp_avg_sq[o:o + s.numel].copy_(st["exp_avg_sq"].reshape(-1))
            self.opt_step = int(float(st["step"]))
        if sd.get("param_groups"):
            for k in ("lr", "betas", "eps", "weight_decay"):
                if k in sd["param_groups"][0]:
                    v = sd["param_groups"][0][k]
                    self.adamw_opt.param_groups[0][k] = tuple(v) if k == "betas" else v
