"""HTTP front end of the serving engine: the reference's routes and payloads
(``serve.py:237-252,489-594``) on top of continuous batching.

Routes: ``GET /health``, ``GET /info``, ``POST /generate`` (JSON, or SSE frames
``data: {"token": ...}`` ... ``data: {"done": true, "prompt_tokens", "completion_tokens"}`` when
``stream`` is set), ``POST /v1/completions`` and ``GET /v1/models`` (OpenAI-compatible;
``frequency_penalty`` maps to ``repetition_penalty = 1 + fp``, ``n <= 8``).  A prompt that does
not fit the context answers 400.

Requests from any number of clients are queued to one worker thread that owns the engine and
calls ``step()`` in a loop, so concurrent requests share decode batches (the reference serves
one request at a time inside its handler).
"""
from __future__ import annotations

import asyncio
import json
import queue
import threading
import time
from typing import Any, Optional, Union

from ..data.tokenizer import ByteTokenizer, load_tokenizer  # noqa: F401  (re-exported: the server's public names)
from .engine import Request, SamplingParams, ServingEngine


from pydantic import BaseModel, Field


class GenerateRequest(BaseModel):
    prompt: str
    max_new_tokens: int = Field(256, ge=1, le=2048)
    temperature: float = Field(0.7, ge=0.0, le=2.0)
    top_k: int = Field(50, ge=0)
    top_p: float = Field(0.0, ge=0.0, le=1.0)
    repetition_penalty: float = Field(1.0, ge=1.0, le=2.0)
    stop_strings: list[str] = Field(default_factory=list)
    stream: bool = False

class GenerateResponse(BaseModel):
    text: str
    prompt_tokens: int
    completion_tokens: int
    tokens_per_second: float

class CompletionRequest(BaseModel):
    model: str = "kotodama"
    prompt: str
    max_tokens: int = Field(256, ge=1, le=2048)
    temperature: float = Field(0.7, ge=0.0, le=2.0)
    top_p: float = Field(0.0, ge=0.0, le=1.0)
    frequency_penalty: float = Field(0.0, ge=0.0, le=1.0)     # becomes repetition_penalty = 1 + this (at most 2, the sampler's limit)
    presence_penalty: float = Field(0.0, ge=0.0, le=2.0)      # accepted for client compatibility, not used (as in the reference)
    best_of: Optional[int] = None                             # accepted, not used
    n: int = Field(1, ge=1, le=8)
    stop: Union[list[str], str, None] = None          # a single string or a list, as the OpenAI API allows



class Ticket:
    """Handle of one submitted request: the queue its tokens arrive on, and what a cancel needs."""

    def __init__(self) -> None:
        self.out: "queue.Queue" = queue.Queue()
        self.rid: Optional[int] = None
        self.cancelled = False


class EngineWorker:
    """Owns the engine on one thread; clients submit prompts and read tokens from per-request queues.
    A client that stops reading (stop string matched, connection closed) cancels its ticket, which
    takes the request out of the engine and frees its KV pages.  An exception in a step is reported
    to every open stream and the affected requests are retired; the thread keeps serving."""

    def __init__(self, engine: ServingEngine) -> None:
        self.engine = engine
        self._inbox: "queue.Queue[tuple]" = queue.Queue()
        self._streams: dict[int, tuple[Request, Ticket, int]] = {}
        self._stop = False
        self.errors = 0
        self._thread = threading.Thread(target=self._run, name="engine", daemon=True)
        self._thread.start()

    def submit(self, prompt: list[int], params: SamplingParams) -> Ticket:
        t = Ticket()
        self._inbox.put(("add", t, prompt, params))
        return t

    def cancel(self, ticket: Ticket) -> None:
        ticket.cancelled = True
        self._inbox.put(("cancel", ticket, None, None))

    def _handle(self, item: tuple) -> None:
        kind, ticket, prompt, params = item
        if kind == "add":
            if ticket.cancelled:
                return
            try:
                r = self.engine.add_request(prompt, params)
                ticket.rid = r.rid
                self._streams[r.rid] = (r, ticket, 0)
            except ValueError as e:
                ticket.out.put(("error", str(e)))
        elif ticket.rid is not None and ticket.rid in self._streams:
            self.engine.cancel(ticket.rid)
            del self._streams[ticket.rid]

    def _drain_inbox(self, block: bool) -> None:
        try:
            item = self._inbox.get(timeout=0.05) if block else self._inbox.get_nowait()
        except queue.Empty:
            return
        while True:
            self._handle(item)
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return

    def _fail_all(self, msg: str) -> None:
        """A step raised: every open stream gets the error, its request leaves the engine."""
        self.errors += 1
        for rid, (r, ticket, _) in list(self._streams.items()):
            ticket.out.put(("error", msg))
            self.engine.cancel(rid)
        self._streams.clear()

    def _run(self) -> None:
        while not self._stop:
            self._drain_inbox(block=not self.engine.has_work())
            if not self.engine.has_work():
                continue
            try:
                self.engine.step()
            except Exception as e:                             # noqa: BLE001 - the worker must outlive a bad step
                self._fail_all(f"{type(e).__name__}: {e}")
                continue
            for rid, (r, ticket, sent) in list(self._streams.items()):
                for t in r.generated[sent:]:
                    ticket.out.put(("token", t))
                self._streams[rid] = (r, ticket, len(r.generated))
                if r.finished:
                    ticket.out.put(("done", r.finish_reason))
                    del self._streams[rid]

    def shutdown(self) -> None:
        self._stop = True
        self._thread.join(timeout=5)


def create_app(engine: ServingEngine, tokenizer: Any = None, model_name: str = "kotodama", checkpoint: str = "",
               trim_stop_strings: bool = False) -> Any:
    """The HTTP application.  A stop string ends a request as in the reference server (``serve.py:375-378,455-457``): the
    text keeps everything up to and including the token that completed the stop string, and the first generated token
    is not checked; ``trim_stop_strings=True`` cuts the text in front of the stop string instead (OpenAI semantics)."""
    from fastapi import FastAPI, HTTPException
    from fastapi.responses import StreamingResponse

    tok = tokenizer or ByteTokenizer()
    worker = EngineWorker(engine)
    app = FastAPI(title="kotodama-b200 inference server")
    app.state.worker = worker

    def params_of(req: GenerateRequest) -> SamplingParams:
        return SamplingParams(max_new_tokens=req.max_new_tokens, temperature=req.temperature, top_k=req.top_k,
                              top_p=req.top_p, repetition_penalty=req.repetition_penalty,
                              eos_token_id=getattr(tok, "eos_token_id", None))

    def encode(prompt: str) -> list[int]:
        ids = list(tok.encode(prompt)) or [0]
        bad = [i for i in ids if not 0 <= i < engine.cfg.vocab_size]
        if bad:
            raise HTTPException(status_code=400, detail=f"tokenizer produced {len(bad)} ids outside the model's "
                                                        f"vocabulary of {engine.cfg.vocab_size} (first: {bad[0]})")
        if len(ids) >= engine.max_ctx:
            raise HTTPException(status_code=400, detail=f"Prompt too long: {len(ids)} tokens >= {engine.max_ctx}")
        return ids

    def collect(ticket: Ticket, stop_strings: list[str]):
        """Blocking generator of (kind, payload, text_so_far).  Leaving it before the engine finished
        the request (stop string, client gone) cancels the request in the engine."""
        ids: list[int] = []
        text = ""
        finished = False
        try:
            while True:
                kind, val = ticket.out.get()
                if kind == "error":
                    finished = True
                    raise HTTPException(status_code=400 if "KV pages" in val or "prompt" in val else 500, detail=val)
                if kind == "done":
                    finished = True
                    yield "done", val, text
                    return
                ids.append(val)
                new_text = tok.decode(ids, skip_special_tokens=True)
                delta, text = new_text[len(text):], new_text
                hit = next((s for s in stop_strings if s and s in text), None) if len(ids) > 1 or trim_stop_strings else None
                if hit is not None and trim_stop_strings:
                    cut = text.index(hit)
                    yield "token", delta[: max(0, len(delta) - (len(text) - cut))], text[:cut]
                    yield "done", "stop", text[:cut]
                    return
                yield "token", delta, text
                if hit is not None:
                    yield "done", "stop", text
                    return
        finally:
            if not finished:
                worker.cancel(ticket)

    @app.get("/health")
    def health() -> dict[str, Any]:
        return {"status": "ok", "running": len(engine.running), "waiting": len(engine.waiting)}

    @app.get("/info")
    def info() -> dict[str, Any]:
        c = engine.cfg
        # the reference's fields (``serve.py:255-262,494-505``: name, params, config, device, checkpoint, fast_attnres),
        # then what this engine adds
        return {"name": model_name, "params": c.param_count(), "config": c.to_dict(), "checkpoint": checkpoint,
                "model": model_name, "hidden_size": c.hidden_size, "num_layers": c.num_layers,
                "vocab_size": c.vocab_size, "max_position_embeddings": c.max_position_embeddings,
                "attn_res": c.attn_res, "fast_attnres": True, "device": str(engine.device),
                "dtype": str(engine.dtype).replace("torch.", ""), "kv_cache": "paged-16",
                "max_batch": engine.max_batch, "tokenizer": getattr(tok, "name", type(tok).__name__)}

    @app.get("/stats")
    def stats() -> dict[str, Any]:
        """Scheduler counters since start-up (not a reference route): tokens and seconds spent in prefill
        and decode, prefill passes (several prompts may share one), steps, free KV pages."""
        return {**engine.stats, "free_pages": len(engine.cache.free), "num_pages": engine.cache.num_pages,
                "running": len(engine.running), "waiting": len(engine.waiting)}

    @app.post("/generate")
    async def generate(req: GenerateRequest):
        ids = encode(req.prompt)
        q = worker.submit(ids, params_of(req))
        loop = asyncio.get_running_loop()
        t0 = time.perf_counter()
        if req.stream:
            async def frames():
                gen = collect(q, req.stop_strings)
                n = 0
                try:
                    while True:
                        kind, val, _ = await loop.run_in_executor(None, next, gen)
                        if kind == "token":
                            n += 1
                            if val:
                                yield f"data: {json.dumps({'token': val})}\n\n"
                        else:
                            yield f"data: {json.dumps({'done': True, 'prompt_tokens': len(ids), 'completion_tokens': n})}\n\n"
                            return
                finally:
                    gen.close()                               # a dropped connection cancels the request
            return StreamingResponse(frames(), media_type="text/event-stream")

        def run() -> tuple[str, int]:
            n, text = 0, ""
            for kind, _, text in collect(q, req.stop_strings):
                n += kind == "token"
            return text, n
        text, n = await loop.run_in_executor(None, run)
        dt = max(time.perf_counter() - t0, 1e-9)
        return GenerateResponse(text=text, prompt_tokens=len(ids), completion_tokens=n, tokens_per_second=n / dt)

    @app.get("/v1/models")
    def models() -> dict[str, Any]:
        return {"object": "list", "data": [{"id": model_name, "object": "model", "owned_by": "kotodama"}]}

    @app.post("/v1/completions")
    async def completions(req: CompletionRequest):
        ids = encode(req.prompt)
        loop = asyncio.get_running_loop()
        sp = SamplingParams(max_new_tokens=req.max_tokens, temperature=req.temperature, top_k=50, top_p=req.top_p,
                            repetition_penalty=1.0 + req.frequency_penalty,
                            eos_token_id=getattr(tok, "eos_token_id", None))
        queues = [worker.submit(ids, sp) for _ in range(req.n)]       # the n samples share decode batches

        def run(q) -> tuple[str, int, str]:
            n, text, reason = 0, "", "length"
            stops = [req.stop] if isinstance(req.stop, str) else (req.stop or [])
            for kind, val, text in collect(q, stops):
                if kind == "token":
                    n += 1
                else:
                    reason = "stop" if val in ("eos", "stop") else "length"
            return text, n, reason
        results = [await loop.run_in_executor(None, run, q) for q in queues]
        total = sum(r[1] for r in results)
        return {"id": f"cmpl-{int(time.time() * 1000)}", "object": "text_completion", "created": int(time.time()),
                "model": model_name,
                "choices": [{"text": t, "index": i, "logprobs": None, "finish_reason": fr}
                            for i, (t, _, fr) in enumerate(results)],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": total, "total_tokens": len(ids) + total}}

    return app
