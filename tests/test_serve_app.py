"""HTTP contract of the server (FastAPI test client, CPU engine, byte tokenizer)."""
import json

import pytest
import torch

from kotodama_b200.config import ModelConfig
from kotodama_b200.models.llama import KotodamaModel
from kotodama_b200.serve.app import ByteTokenizer, create_app
from kotodama_b200.serve.engine import ServingEngine

fastapi = pytest.importorskip("fastapi")
from fastapi.testclient import TestClient  # noqa: E402


@pytest.fixture(scope="module")
def client():
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_attention_heads=2, num_kv_heads=1, head_dim=32,
                      intermediate_size=96, vocab_size=300, max_position_embeddings=64, attn_res=True,
                      attn_res_n_blocks=2)
    eng = ServingEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32, max_batch=4, max_ctx=64)
    app = create_app(eng, ByteTokenizer(), model_name="test")
    with TestClient(app) as c:
        yield c
    app.state.worker.shutdown()


def test_health_info_models(client):
    assert client.get("/health").json()["status"] == "ok"
    info = client.get("/info").json()
    assert info["attn_res"] is True and info["kv_cache"] == "paged-16" and "fast_attnres" in info
    assert client.get("/v1/models").json()["data"][0]["id"] == "test"


def test_generate_json_and_limits(client):
    r = client.post("/generate", json={"prompt": "hello", "max_new_tokens": 5, "temperature": 0})
    body = r.json()
    assert r.status_code == 200 and body["prompt_tokens"] == 5 and 1 <= body["completion_tokens"] <= 5
    assert set(body) == {"text", "prompt_tokens", "completion_tokens", "tokens_per_second"}
    again = client.post("/generate", json={"prompt": "hello", "max_new_tokens": 5, "temperature": 0}).json()
    assert again["text"] == body["text"]                      # greedy is deterministic
    st = client.get("/stats").json()
    assert st["prefill_tokens"] >= 10 and st["prefill_passes"] >= 2 and st["free_pages"] == st["num_pages"]
    assert client.post("/generate", json={"prompt": "x" * 80}).status_code == 400
    assert client.post("/generate", json={"prompt": "x", "temperature": 3.0}).status_code == 422


def test_generate_stream_frames(client):
    with client.stream("POST", "/generate", json={"prompt": "abc", "max_new_tokens": 4, "temperature": 0,
                                                  "stream": True}) as r:
        frames = [json.loads(l[6:]) for l in r.iter_lines() if l.startswith("data: ")]
    assert frames[-1]["done"] is True and frames[-1]["prompt_tokens"] == 3
    assert 1 <= frames[-1]["completion_tokens"] <= 4
    assert all("token" in f for f in frames[:-1])


def test_openai_completions(client):
    r = client.post("/v1/completions", json={"prompt": "hi", "max_tokens": 3, "n": 2, "temperature": 0,
                                             "frequency_penalty": 0.5})
    body = r.json()
    assert r.status_code == 200 and len(body["choices"]) == 2 and body["object"] == "text_completion"
    assert body["usage"]["prompt_tokens"] == 2 and body["usage"]["completion_tokens"] <= 6
    assert client.post("/v1/completions", json={"prompt": "hi", "n": 9}).status_code == 422


def test_stop_as_string_cancels_the_request_in_the_engine(client):
    """OpenAI clients may send ``stop`` as one string; a stop hit ends the request in the engine too
    (its KV pages come back although max_tokens was not reached)."""
    import time
    full = client.post("/v1/completions", json={"prompt": "hi", "max_tokens": 40, "temperature": 0}).json()
    text = full["choices"][0]["text"]
    stop = next((ch for ch in text[1:] if ch.strip()), None)
    if stop is None:
        pytest.skip("model produced no printable character to stop on")
    r = client.post("/v1/completions", json={"prompt": "hi", "max_tokens": 40, "temperature": 0, "stop": stop})
    body = r.json()
    got = body["choices"][0]["text"]
    # as in the reference server the text runs up to and including the stop string (looked for from the second token on)
    assert r.status_code == 200 and got.endswith(stop) and len(got) < len(text) and body["choices"][0]["finish_reason"] == "stop"
    assert stop not in got[1:-len(stop)]
    for _ in range(100):                                      # the cancel travels through the worker's inbox
        st = client.get("/stats").json()
        if st["free_pages"] == st["num_pages"] and st["running"] == 0:
            break
        time.sleep(0.02)
    assert st["free_pages"] == st["num_pages"] and st["running"] == 0


def test_worker_survives_a_failing_step(client):
    """An exception inside a step reaches the waiting client as an error and the worker keeps serving."""
    worker = client.app.state.worker
    eng = worker.engine
    real = eng.step
    calls = {"n": 0}

    def boom():
        calls["n"] += 1
        raise RuntimeError("KV cache exhausted")
    eng.step = boom
    try:
        r = client.post("/generate", json={"prompt": "hello", "max_new_tokens": 5, "temperature": 0})
        assert r.status_code == 500 and "KV cache exhausted" in r.json()["detail"]
    finally:
        eng.step = real
    assert calls["n"] == 1 and worker.errors == 1 and not eng.has_work()
    ok = client.post("/generate", json={"prompt": "hello", "max_new_tokens": 3, "temperature": 0})
    assert ok.status_code == 200 and ok.json()["completion_tokens"] >= 1


def test_trimmed_stop_strings_are_an_option():
    """``trim_stop_strings=True``: the text ends in front of the stop string, and the first token is checked too."""
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_attention_heads=2, num_kv_heads=1, head_dim=32,
                      intermediate_size=96, vocab_size=300, max_position_embeddings=64)
    eng = ServingEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32, max_batch=2, max_ctx=64)
    app = create_app(eng, ByteTokenizer(), model_name="test", trim_stop_strings=True)
    with TestClient(app) as c:
        text = c.post("/generate", json={"prompt": "hi", "max_new_tokens": 30, "temperature": 0}).json()["text"]
        stop = next((ch for ch in text if ch.strip()), None)
        if stop is None:
            pytest.skip("model produced no printable character to stop on")
        got = c.post("/generate", json={"prompt": "hi", "max_new_tokens": 30, "temperature": 0, "stop_strings": [stop]}).json()["text"]
        assert got == text[: text.index(stop)]
    app.state.worker.shutdown()
