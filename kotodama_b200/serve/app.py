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
from typing import Any, Optional

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
    frequency_penalty: float = Field(0.0, ge=0.0, le=1.0)
    n: int = Field(1, ge=1, le=8)
    stop: Optional[list[str]] = None


class ByteTokenizer:
    """Fallback tokenizer (UTF-8 bytes + BOS/EOS) used when no Hugging Face tokenizer files are
    available offline.  ids 0..255 are bytes, 256 = BOS, 257 = EOS."""

    bos_token_id, eos_token_id, vocab_size = 256, 257, 258
    name = "bytes"

    def encode(self, text: str) -> list[int]:
        return list(text.encode("utf-8"))

    def decode(self, ids: list[int], skip_special_tokens: bool = True) -> str:
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")


def load_tokenizer(name: Optional[str]) -> Any:
    """Hugging Face tokenizer from local files when present (the reference uses
    ``HuggingFaceTB/SmolLM2-135M``, ``serve.py:227-230``); the byte tokenizer otherwise."""
    if name:
        try:
            from transformers import AutoTokenizer
            return AutoTokenizer.from_pretrained(name, local_files_only=True)
        except Exception:       # noqa: BLE001 - no network / no files
            pass
    return ByteTokenizer()


class EngineWorker:
    """Owns the engine on one thread; clients submit prompts and read tokens from per-request queues."""

    def __init__(self, engine: ServingEngine) -> None:
        self.engine = engine
        self._inbox: "queue.Queue[tuple[list[int], SamplingParams, queue.Queue]]" = queue.Queue()
        self._streams: dict[int, tuple[Request, "queue.Queue", int]] = {}
        self._stop = False
        self._thread = threading.Thread(target=self._run, name="engine", daemon=True)
        self._thread.start()

    def submit(self, prompt: list[int], params: SamplingParams) -> "queue.Queue":
        out: "queue.Queue" = queue.Queue()
        self._inbox.put((prompt, params, out))
        return out

    def _drain_inbox(self, block: bool) -> None:
        try:
            item = self._inbox.get(timeout=0.05) if block else self._inbox.get_nowait()
        except queue.Empty:
            return
        while True:
            prompt, params, out = item
            try:
                r = self.engine.add_request(prompt, params)
                self._streams[r.rid] = (r, out, 0)
            except ValueError as e:
                out.put(("error", str(e)))
            try:
                item = self._inbox.get_nowait()
            except queue.Empty:
                return

    def _run(self) -> None:
        while not self._stop:
            self._drain_inbox(block=not self.engine.has_work())
            if not self.engine.has_work():
                continue
            self.engine.step()
            for rid, (r, out, sent) in list(self._streams.items()):
                for t in r.generated[sent:]:
                    out.put(("token", t))
                self._streams[rid] = (r, out, len(r.generated))
                if r.finished:
                    out.put(("done", r.finish_reason))
                    del self._streams[rid]

    def shutdown(self) -> None:
        self._stop = True
        self._thread.join(timeout=5)


def create_app(engine: ServingEngine, tokenizer: Any = None, model_name: str = "kotodama") -> Any:
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
        ids = tok.encode(prompt)
        ids = [i for i in ids if i < engine.cfg.vocab_size] or [0]
        if len(ids) >= engine.max_ctx:
            raise HTTPException(status_code=400, detail=f"Prompt too long: {len(ids)} tokens >= {engine.max_ctx}")
        return ids

    def collect(q: "queue.Queue", stop_strings: list[str]):
        """Blocking generator of (kind, payload, text_so_far)."""
        ids: list[int] = []
        text = ""
        while True:
            kind, val = q.get()
            if kind == "error":
                raise HTTPException(status_code=400, detail=val)
            if kind == "done":
                yield "done", val, text
                return
            ids.append(val)
            new_text = tok.decode(ids, skip_special_tokens=True)
            delta, text = new_text[len(text):], new_text
            hit = next((s for s in stop_strings if s and s in text), None)
            if hit is not None:
                cut = text.index(hit)
                yield "token", delta[: max(0, len(delta) - (len(text) - cut))], text[:cut]
                yield "done", "stop", text[:cut]
                return
            yield "token", delta, text

    @app.get("/health")
    def health() -> dict[str, Any]:
        return {"status": "ok", "running": len(engine.running), "waiting": len(engine.waiting)}

    @app.get("/info")
    def info() -> dict[str, Any]:
        c = engine.cfg
        return {"model": model_name, "hidden_size": c.hidden_size, "num_layers": c.num_layers,
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
                while True:
                    kind, val, _ = await loop.run_in_executor(None, next, gen)
                    if kind == "token":
                        n += 1
                        if val:
                            yield f"data: {json.dumps({'token': val})}\n\n"
                    else:
                        yield f"data: {json.dumps({'done': True, 'prompt_tokens': len(ids), 'completion_tokens': n})}\n\n"
                        return
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
            for kind, val, text in collect(q, req.stop or []):
                if kind == "token":
                    n += 1
                else:
                    reason = "stop" if val in ("eos", "stop") else "length"
            return text, n, reason
        results = [await loop.run_in_executor(None, run, q) for q in queues]
        total = sum(r[1] for r in results)
        return {"id": f"cmpl-{int(time.time() * 1000)}", "object": "text_completion", "created": int(time.time()),
                "model": req.model,
                "choices": [{"text": t, "index": i, "logprobs": None, "finish_reason": fr}
                            for i, (t, _, fr) in enumerate(results)],
                "usage": {"prompt_tokens": len(ids), "completion_tokens": total, "total_tokens": len(ids) + total}}

    return app
