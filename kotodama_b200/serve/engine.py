"""Serving engine: paged KV cache (16-token pages), continuous batching, greedy / sampled
decoding on the device.

The reference server (``serve.py:322-391``) handles one request at a time with a contiguous KV
cache grown by ``torch.cat``.  Here any number of requests run concurrently: a request is
prefilled in one pass over its prompt (writing post-norm, post-RoPE keys and values straight
into its pages; requests admitted in the same step share that pass, packed back to back with
the attention kernel taking the sequence boundaries), then joins the decode batch, where every step advances all running requests
by one token with the split-KV paged attention kernel.  Pages return to the free list when a
request finishes.

AttnRes needs no cross-token state at inference: the sources of a routing call are that
token's own block summaries, rebuilt layer by layer (``src/model/llama.py:718-763``), so only
keys and values are cached.

The layer pipeline is the executor's forward schedule (same ops backend: PyTorch on CPU,
sm_100a kernels on CUDA); sampling follows the reference order repetition penalty ->
temperature -> top-k -> top-p -> multinomial, greedy at temperature 0 (``serve.py:266-304``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Any, Optional

import numpy as np
import torch

from ..config import ModelConfig
from ..engine import ParamArena
from ..models.llama import KotodamaModel
from ..ops import get_ops

PAGE = 16


@dataclass
class SamplingParams:
    max_new_tokens: int = 256
    temperature: float = 0.7
    top_k: int = 50
    top_p: float = 0.0
    repetition_penalty: float = 1.0
    eos_token_id: Optional[int] = None
    seed: Optional[int] = None           # of the sampler's random draws; None: derived from the request id


@dataclass
class Request:
    rid: int
    prompt: list[int]
    params: SamplingParams
    pages: list[int] = field(default_factory=list)
    generated: list[int] = field(default_factory=list)
    ctx_len: int = 0
    finished: bool = False
    finish_reason: str = ""
    slot: int = -1                       # row of the engine's seen-token bitmap (repetition penalty)


class PagedKVCache:
    """Per-layer key/value page pools and a free list shared by all layers (a page index means
    the same slot in every layer)."""

    def __init__(self, cfg: ModelConfig, num_pages: int, device: torch.device, dtype: torch.dtype,
                 n_kv_local: Optional[int] = None) -> None:
        self.n_kv = n_kv_local or cfg.num_kv_heads
        self.hd = cfg.head_dim
        self.num_pages = num_pages
        shape = (cfg.num_layers, num_pages, self.n_kv, PAGE, self.hd)      # 16 rows of one (page, head) are contiguous
        self.k = torch.zeros(shape, device=device, dtype=dtype)
        self.v = torch.zeros(shape, device=device, dtype=dtype)
        self.free = list(range(num_pages - 1, -1, -1))

    def pages_for(self, tokens: int) -> int:
        return (tokens + PAGE - 1) // PAGE

    def can_allocate(self, n: int) -> bool:
        return len(self.free) >= n

    def allocate(self, n: int) -> list[int]:
        if len(self.free) < n:
            raise RuntimeError("KV cache exhausted")
        return [self.free.pop() for _ in range(n)]

    def release(self, pages: list[int]) -> None:
        self.free.extend(reversed(pages))


def request_seed(r: Request) -> int:
    return r.params.seed if r.params.seed is not None else (0x9E3779B1 * (r.rid + 1) + 12345) & 0x7FFFFFFF


def sample_tokens(logits: torch.Tensor, reqs: list[Request], ops: Any, seen: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Next token per row of ``logits[B,V]``.  All-greedy batches use the argmax kernel; anything else
    goes to the batched sampler of the ops backend (on CUDA one kernel for the whole batch, with
    per-request parameters, seeds and seen-token bitmaps): repetition penalty -> temperature -> top-k
    -> top-p -> multinomial, the reference's order (``serve.py:266-304``)."""
    if all(r.params.temperature == 0 and r.params.repetition_penalty == 1.0 for r in reqs):
        return ops.argmax(logits)
    ps = [r.params for r in reqs]
    slots = [max(r.slot, 0) for r in reqs]
    if seen is None and any(p.repetition_penalty != 1.0 for p in ps):
        # no engine-owned bitmaps (direct use): build them from the requests' token lists
        import numpy as np
        words = np.zeros((len(reqs), (logits.shape[1] + 31) // 32), dtype=np.uint32)
        for b, r in enumerate(reqs):                     # generated tokens only, as the reference's server counts them
            ids = np.unique(np.asarray(r.generated, dtype=np.int64))
            np.bitwise_or.at(words[b], ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
        seen = torch.from_numpy(words.view(np.int32)).to(logits.device)
        slots = list(range(len(reqs)))
    return ops.sample(logits, [p.temperature for p in ps], [p.top_k for p in ps], [p.top_p for p in ps],
                      [p.repetition_penalty for p in ps], [request_seed(r) for r in reqs],
                      [len(r.generated) for r in reqs], seen, slots)


class ServingEngine:
    def __init__(self, model: KotodamaModel, *, device: torch.device | str = "cpu",
                 dtype: torch.dtype = torch.float32, max_batch: int = 64, num_pages: Optional[int] = None,
                 max_ctx: Optional[int] = None, ops: Any = None, tp: Any = None,
                 prefill_batch_tokens: int = 8192) -> None:
        self.device = torch.device(device)
        self.dtype = dtype
        self.model = model.eval()
        self.cfg: ModelConfig = model.config
        self.ops = ops or get_ops(self.device)
        self.tp = tp                                  # tensor-parallel helper (``serve.tp``) or None
        if tp is not None:
            tp.prepare_model(model)
        self.arena = ParamArena(model, self.device, dtype, with_grads=False)
        cfg = self.cfg
        self.max_ctx = max_ctx or cfg.max_position_embeddings
        self.max_batch = max_batch
        tpn = tp.size if tp is not None else 1
        self.H, self.KV = cfg.num_attention_heads // tpn, cfg.num_kv_heads // tpn
        self.hd, self.D = cfg.head_dim, cfg.hidden_size
        pages = num_pages or max_batch * ((self.max_ctx + PAGE - 1) // PAGE)
        self.cache = PagedKVCache(cfg, pages, self.device, dtype, n_kv_local=self.KV)
        self.max_pages_per_req = (self.max_ctx + PAGE - 1) // PAGE
        self.waiting: list[Request] = []
        self.running: list[Request] = []
        self._next_id = 0
        # one bitmap row per batch slot: the tokens a request has generated so far, for the repetition penalty of
        # the device sampler (the reference's server penalises generated tokens only, ``serve.py:266-283,345-373``;
        # ``penalise_prompt`` adds the prompt's tokens, the convention of other serving stacks)
        self.penalise_prompt = False
        self.seen_words = (cfg.vocab_size + 31) // 32
        self.seen = torch.zeros(max_batch, self.seen_words, dtype=torch.int32, device=self.device)
        self._free_slots = list(range(max_batch - 1, -1, -1))
        self._dec_states: dict[int, dict] = {}
        self.use_cuda_graphs = True          # decode steps are replayed from captured graphs on CUDA
        # captured decode kernels start while the kernel before them drains (KOTODAMA_DEPENDENT_LAUNCH=0: plain order)
        self.dependent_launch = os.environ.get("KOTODAMA_DEPENDENT_LAUNCH", "1") != "0"
        self.graph_ms: Optional[list[float]] = None      # set to a list to collect the device time of every decode replay
        self._graph_events: list = []
        # when a list: every pass appends ([request ids], fp32 logits on the host) - for tests that compare
        # two engines by logits rather than by sampled tokens
        self.logit_trace: Optional[list] = None
        self.prefill_batch_tokens = prefill_batch_tokens     # tokens of one packed prefill pass over several prompts; 0: one prompt per pass
        self.stats = {"prefill_tokens": 0, "decode_tokens": 0, "prefill_s": 0.0, "decode_s": 0.0, "steps": 0,
                      "prefill_passes": 0}
        ar = self.arena
        self.layers = []
        for i in range(cfg.num_layers):
            p = f"layers.{i}."
            g = lambda n: ar.view(p + n) if (p + n) in ar.by_name else None
            dw = self.ops.decode_weight          # on CUDA: adds the tile-major copy that decode-size products stream
            self.layers.append(dict(
                wqkv=dw(ar.fused(p + "attn.q_proj.weight", p + "attn.v_proj.weight")), wo=dw(ar.view(p + "attn.o_proj.weight")),
                wgu=dw(ar.fused(p + "ffn.gate_proj.weight", p + "ffn.up_proj.weight")), wd=dw(ar.view(p + "ffn.down_proj.weight")),
                attn_norm=g("attn_norm.weight"), ffn_norm=g("ffn_norm.weight"), qn=g("attn.q_norm.weight"),
                kn=g("attn.k_norm.weight"), aq=g("attn_res_query"), an=g("attn_res_norm.weight"),
                mq=g("mlp_res_query"), mn=g("mlp_res_norm.weight")))
        self.boundaries = frozenset(cfg.boundaries()) if cfg.attn_res else frozenset()

    # ------------------------------------------------------------------ requests
    def add_request(self, prompt: list[int], params: Optional[SamplingParams] = None) -> Request:
        params = params or SamplingParams()
        if len(prompt) == 0:
            raise ValueError("empty prompt")
        if len(prompt) + 1 > self.max_ctx:
            raise ValueError(f"prompt of {len(prompt)} tokens does not fit the context of {self.max_ctx}")
        need = self.cache.pages_for(min(len(prompt) + params.max_new_tokens, self.max_ctx))
        if need > self.cache.num_pages:
            raise ValueError(f"request needs {need} KV pages, the cache has {self.cache.num_pages}")
        r = Request(self._next_id, list(prompt), params)
        self._next_id += 1
        self.waiting.append(r)
        return r

    def cancel(self, rid: int) -> bool:
        """Ends request ``rid`` now (a client went away, a stop string matched): it leaves the waiting
        queue or the decode batch and its KV pages return to the free list.  Call between steps."""
        for lst in (self.waiting, self.running):
            for r in lst:
                if r.rid == rid:
                    lst.remove(r)
                    self._release(r)
                    r.finished, r.finish_reason = True, "cancelled"
                    return True
        return False

    def has_work(self) -> bool:
        return bool(self.waiting or self.running)

    # ------------------------------------------------------------------ model pass
    @torch.no_grad()
    def _forward(self, ids: torch.Tensor, positions: torch.Tensor, slots: torch.Tensor, decode: Optional[dict],
                 last_rows: torch.Tensor, seqs: Optional[dict] = None) -> torch.Tensor:
        """Runs all layers on ``ids[N]``; keys/values go to ``slots`` (negative = padding, dropped).
        ``decode`` holds the page table and context lengths for paged attention; ``None`` means a
        causal prefill of ``prompts`` requests, each padded to ``N / prompts`` rows.
        Returns logits for ``last_rows``."""
        ops, cfg, ar = self.ops, self.cfg, self.arena
        H, KV, hd = self.H, self.KV, self.hd
        eps = cfg.norm_eps
        cos, sin = self.model.rope_cos, self.model.rope_sin
        N = ids.numel()
        x = ops.embedding_fwd(ids, ar.view("embed_tokens.weight"))
        committed: list[torch.Tensor] = []
        partial: Optional[torch.Tensor] = x
        for i, lw in enumerate(self.layers):
            xn, _ = ops.route_norm_fwd(committed + [partial], lw["aq"], lw["an"], lw["attn_norm"], eps)
            if i in self.boundaries:
                committed = committed + [partial]
                partial = None
            qkv = ops.gemm_nt(xn, lw["wqkv"])
            # QK-norm + RoPE; the same launch puts the new keys and values into their cache slots
            qk, _ = ops.qknorm_rope_fwd(qkv, lw["qn"], lw["kn"], cos, sin, N, H, KV, hd, eps, positions=positions,
                                        append=(self.cache.k[i], self.cache.v[i], slots))
            k_rows = qk[:, H * hd:]
            v_rows = qkv[:, (H + KV) * hd:]
            if decode is None:
                o, _ = ops.attention_fwd(qk[:, : H * hd].view(1, N, H, hd), k_rows.view(1, N, KV, hd),
                                         v_rows.view(1, N, KV, hd), need_grad=False, **seqs)
                attn = o.reshape(N, H * hd)
            else:
                attn = ops.paged_decode_attention(qk[:, : H * hd], self.cache.k[i], self.cache.v[i],
                                                  decode["page_table"], decode["ctx_lens"], decode["max_ctx"], H, KV, hd)
            partial = self._row_linear(attn, lw["wo"], partial)
            xn2, _ = ops.route_norm_fwd(committed + [partial], lw["mq"], lw["mn"], lw["ffn_norm"], eps)
            act = ops.swiglu_fwd(ops.gemm_nt(xn2, lw["wgu"]))
            partial = self._row_linear(act, lw["wd"], partial)
        g = lambda n: ar.view(n) if n in ar.by_name else None
        xf, _ = ops.route_norm_fwd([s[last_rows] for s in committed + [partial]], g("final_res_query"),
                                   g("final_res_norm.weight"), ar.view("norm.weight"), eps)
        return ops.gemm_nt(xf, self.model.get_lm_head_weight())

    def _row_linear(self, x: torch.Tensor, w: torch.Tensor, residual: Optional[torch.Tensor]) -> torch.Tensor:
        if self.tp is None:
            return self.ops.gemm_nt(x, w, residual=residual)
        return self.tp.row_linear(self.ops, x, w, residual)

    # ------------------------------------------------------------------ scheduling
    def _prefill(self, reqs: list[Request]) -> None:
        """One pass over the prompts of ``reqs``, packed back to back (no padding): the attention kernel
        takes the sequence boundaries (``cu_seqlens``), every other op is per token."""
        ns = [len(r.prompt) for r in reqs]
        total = sum(ns)
        ids = torch.empty(total, dtype=torch.long)
        slots = torch.empty(total, dtype=torch.long)
        pos = torch.empty(total, dtype=torch.int32)
        cu = [0]
        for r, n in zip(reqs, ns):
            at = cu[-1]
            ids[at:at + n] = torch.tensor(r.prompt, dtype=torch.long)
            t = torch.arange(n)
            slots[at:at + n] = torch.tensor(r.pages, dtype=torch.long)[t // PAGE] * PAGE + t % PAGE
            pos[at:at + n] = t.to(torch.int32)
            cu.append(at + n)
        last = torch.tensor([c - 1 for c in cu[1:]])
        dev = self.device
        seqs = {"cu_seqlens": torch.tensor(cu, dtype=torch.int32).to(dev), "max_seqlen": max(ns)}
        logits = self._forward(ids.to(dev), pos.to(dev), slots.to(dev), None, last.to(dev), seqs=seqs)
        if self.logit_trace is not None:
            self.logit_trace.append(([r.rid for r in reqs], logits.float().cpu()))
        toks = sample_tokens(logits, reqs, self.ops, self.seen).tolist()
        if self.tp is not None:
            toks = self.tp.sync_tokens(toks, self.device)
        for r, n, tok in zip(reqs, ns, toks):
            r.ctx_len = n
            self._accept(r, int(tok))
        self.stats["prefill_tokens"] += total
        self.stats["prefill_passes"] += 1

    def _admit(self) -> list[list[Request]]:
        """Moves the waiting requests that fit (batch slots, pages) to ``running`` and groups them
        into prefill passes of at most ``prefill_batch_tokens`` packed tokens (0: one prompt per pass)."""
        admitted: list[Request] = []
        while self.waiting and len(self.running) < self.max_batch:
            r = self.waiting[0]
            need = self.cache.pages_for(min(len(r.prompt) + r.params.max_new_tokens, self.max_ctx))
            if not self.cache.can_allocate(need):
                break
            # pages are handed out in admission order, which is also the order of the decode batch:
            # neighbouring requests of a decode step then read neighbouring pages
            r.pages = self.cache.allocate(need)
            r.slot = self._free_slots.pop()
            if r.params.repetition_penalty != 1.0:
                self._init_seen(r)
            self.waiting.pop(0)
            self.running.append(r)
            admitted.append(r)
        groups: list[list[Request]] = []
        cur: list[Request] = []
        for r in admitted:
            if cur and sum(len(q.prompt) for q in cur) + len(r.prompt) > self.prefill_batch_tokens:
                groups.append(cur)
                cur = []
            cur.append(r)
        if cur:
            groups.append(cur)
        return groups

    def _init_seen(self, r: Request) -> None:
        """A fresh bitmap row for the request's slot: empty (the sampler sets a bit per generated token), or the
        prompt's tokens when ``penalise_prompt`` is on."""
        words = np.zeros(self.seen_words, dtype=np.uint32)
        if self.penalise_prompt:
            ids = np.unique(np.asarray(r.prompt, dtype=np.int64))
            np.bitwise_or.at(words, ids >> 5, (np.uint32(1) << (ids & 31).astype(np.uint32)))
        self.seen[r.slot].copy_(torch.from_numpy(words.view(np.int32)), non_blocking=True)

    def _release(self, r: Request) -> None:
        if r.pages:
            self.cache.release(r.pages)
            r.pages = []
        if r.slot >= 0:
            self._free_slots.append(r.slot)
            r.slot = -1

    def _accept(self, r: Request, tok: int) -> None:
        r.generated.append(tok)
        p = r.params
        if p.eos_token_id is not None and tok == p.eos_token_id:
            r.finished, r.finish_reason = True, "eos"
        elif len(r.generated) >= p.max_new_tokens:
            r.finished, r.finish_reason = True, "length"
        elif r.ctx_len + 1 >= self.max_ctx:
            r.finished, r.finish_reason = True, "context"

    def _decode_inputs(self, reqs: list[Request]):
        """Static device buffers for a decode step; the page table is rebuilt only when the set of
        running requests changes (pages are assigned once, at admission)."""
        B = len(reqs)
        key = tuple(r.rid for r in reqs)
        # static buffers and captured graphs are kept per batch size: a batch size that comes back
        # (requests of unequal length retire one by one) replays its old graphs
        st = self._dec_states.get(B)
        if st is None:
            # ids | slots (int64), pos | ctx (int32) live in ONE device buffer with a pinned host twin: a decode
            # step costs one host -> device copy of 24 bytes per request
            dev = self.device
            packed = torch.zeros(24 * B, dtype=torch.uint8, device=dev)
            host = torch.zeros(24 * B, dtype=torch.uint8, pin_memory=dev.type == "cuda")
            cut = lambda t, lo, hi, dt: t[lo * B: hi * B].view(dt)
            st = {"B": B, "key": None, "packed": packed, "host": host,
                  "ids": cut(packed, 0, 8, torch.long), "slots": cut(packed, 8, 16, torch.long),
                  "pos": cut(packed, 16, 20, torch.int32), "ctx": cut(packed, 20, 24, torch.int32),
                  "h_ids": cut(host, 0, 8, torch.long).numpy(), "h_slots": cut(host, 8, 16, torch.long).numpy(),
                  "h_pos": cut(host, 16, 20, torch.int32).numpy(), "h_ctx": cut(host, 20, 24, torch.int32).numpy(),
                  "table": torch.zeros(B, self.max_pages_per_req, dtype=torch.int32, device=dev),
                  "rows": torch.arange(B, device=dev), "idx": np.arange(B), "graphs": {}}
            self._dec_states[B] = st
        if st["key"] != key:
            table = np.zeros((B, self.max_pages_per_req), dtype=np.int32)
            for i, r in enumerate(reqs):
                table[i, : len(r.pages)] = r.pages
            st["table"].copy_(torch.from_numpy(table), non_blocking=True)
            st["host_table"] = table
            st["key"] = key
        lens = np.fromiter((r.ctx_len for r in reqs), dtype=np.int64, count=B)
        st["h_ids"][:] = np.fromiter((r.generated[-1] for r in reqs), dtype=np.int64, count=B)
        st["h_slots"][:] = st["host_table"][st["idx"], lens // PAGE].astype(np.int64) * PAGE + lens % PAGE
        st["h_pos"][:] = lens
        st["h_ctx"][:] = lens + 1
        st["packed"].copy_(st["host"], non_blocking=True)
        return st

    def _decode(self) -> None:
        reqs = self.running
        B = len(reqs)
        st = self._decode_inputs(reqs)
        max_ctx = max(r.ctx_len for r in reqs) + 1
        bucket = min(self.max_ctx, ((max_ctx + 511) // 512) * 512)       # grid of the split-KV kernel
        decode = {"page_table": st["table"], "ctx_lens": st["ctx"], "max_ctx": bucket}
        greedy = all(r.params.temperature == 0 and r.params.repetition_penalty == 1.0 for r in reqs)
        if self.device.type == "cuda" and self.use_cuda_graphs:
            g = st["graphs"].get(bucket)
            if g is None:
                # one eager pass first: lazy initialisation must not happen under capture
                self._forward(st["ids"], st["pos"], st["slots"], decode, st["rows"])
                torch.cuda.synchronize()
                graph = torch.cuda.CUDAGraph()
                # the captured launches are programmatic dependents of one another (the graph keeps the edges)
                with torch.cuda.graph(graph), self.ops.dependent_launch(self.dependent_launch):
                    logits = self._forward(st["ids"], st["pos"], st["slots"], decode, st["rows"])
                    toks = self.ops.argmax(logits)
                g = st["graphs"][bucket] = (graph, logits, toks)
            if self.graph_ms is not None:            # device time of the replay alone (what the host adds is wall - this)
                ev = (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True))
                ev[0].record()
                g[0].replay()
                ev[1].record()
                self._graph_events.append(ev)
            else:
                g[0].replay()
            logits, toks = g[1], g[2]
            toks = toks if greedy else sample_tokens(logits, reqs, self.ops, self.seen)
        else:
            logits = self._forward(st["ids"], st["pos"], st["slots"], decode, st["rows"])
            toks = sample_tokens(logits, reqs, self.ops, self.seen)
        if self.logit_trace is not None:
            self.logit_trace.append(([r.rid for r in reqs], logits[:B].float().cpu()))
        # one device -> host read per step (under tensor parallelism: of rank 0's tokens, broadcast on the device)
        toks = self.tp.sync_tokens(toks, self.device) if self.tp is not None else toks.tolist()
        if self.graph_ms is not None and self._graph_events:
            self.graph_ms += [a.elapsed_time(b) for a, b in self._graph_events]     # the token read above synchronised
            self._graph_events.clear()
        for r, t in zip(reqs, toks):
            r.ctx_len += 1
            self._accept(r, int(t))
        self.stats["decode_tokens"] += B

    def step(self) -> list[Request]:
        """Admit and prefill what fits, advance every running request by one token, retire the
        finished.  Returns the requests that finished in this step."""
        import time
        t0 = time.perf_counter()
        for group in self._admit():
            self._prefill(group)
        t1 = time.perf_counter()
        live = [r for r in self.running if not r.finished]
        done = [r for r in self.running if r.finished]
        self.running = live
        if live:
            self._decode()
        done += [r for r in self.running if r.finished]
        self.running = [r for r in self.running if not r.finished]
        for r in done:
            self._release(r)
        self.stats["prefill_s"] += t1 - t0
        self.stats["decode_s"] += time.perf_counter() - t1
        self.stats["steps"] += 1
        return done

    def generate(self, prompts: list[list[int]], params: Optional[SamplingParams] = None) -> list[list[int]]:
        """Convenience: run a set of prompts to completion; returns the generated ids per prompt."""
        reqs = [self.add_request(p, params) for p in prompts]
        while self.has_work():
            self.step()
        return [r.generated for r in reqs]
