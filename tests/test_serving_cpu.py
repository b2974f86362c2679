"""Paged-KV continuous-batching engine against the plain model (contiguous KV cache, one request)."""
import pytest
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.models.llama import KotodamaModel
from kotodama_b200.serve.engine import PagedKVCache, SamplingParams, ServingEngine, sample_tokens, Request


def _model(attn_res=True):
    torch.manual_seed(0)
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=attn_res, attn_res_n_blocks=2)
    m = KotodamaModel(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "query" in n:
                p.normal_(0, 0.3)
    return cfg, m


def _greedy_reference(model, prompt, n_new):
    ids = torch.tensor([prompt])
    out = model(ids, use_cache=True)
    past, toks = out["past_kv"], []
    nxt = int(out["logits"][0, -1].argmax())
    toks.append(nxt)
    for _ in range(n_new - 1):
        out = model(torch.tensor([[nxt]]), use_cache=True, past_kv=past)
        past = out["past_kv"]
        nxt = int(out["logits"][0, -1].argmax())
        toks.append(nxt)
    return toks


def test_paged_engine_matches_contiguous_cache_greedy():
    import copy
    for attn_res in (True, False):
        cfg, model = _model(attn_res)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (5, 17, 33, 16)]
        ref = [_greedy_reference(model, p, 12) for p in prompts]
        eng = ServingEngine(copy.deepcopy(model), device="cpu", dtype=torch.float32, max_batch=3, max_ctx=128)
        got = eng.generate(prompts, SamplingParams(max_new_tokens=12, temperature=0.0))
        assert got == ref
        assert len(eng.cache.free) == eng.cache.num_pages          # every page returned
        assert eng.stats["prefill_tokens"] == sum(map(len, prompts))


def test_prompts_share_a_packed_prefill_pass():
    """Prompts admitted together run as one packed pass (sequence boundaries go to the attention
    kernel, nothing is padded), however unequal their lengths; the token budget splits passes."""
    import copy
    cfg, model = _model()
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 33, 28, 31, 9)]
    ref = [_greedy_reference(model, p, 6) for p in prompts]
    eng = ServingEngine(copy.deepcopy(model), device="cpu", dtype=torch.float32, max_batch=8, max_ctx=128)
    got = eng.generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.0))
    assert got == ref
    assert eng.stats["prefill_passes"] == 1
    eng.prefill_batch_tokens = 64                                  # 30+33 | 28+31 | 9
    eng.stats["prefill_passes"] = 0
    assert eng.generate(prompts, SamplingParams(max_new_tokens=6, temperature=0.0)) == ref
    assert eng.stats["prefill_passes"] == 3


def test_cancel_releases_pages_and_oversize_requests_are_refused():
    cfg, model = _model()
    eng = ServingEngine(model, device="cpu", dtype=torch.float32, max_batch=4, num_pages=8, max_ctx=256)
    with pytest.raises(ValueError):                                 # 10 pages can never be had from a cache of 8
        eng.add_request(list(range(1, 60)), SamplingParams(max_new_tokens=100, temperature=0.0))
    a = eng.add_request([1, 2, 3], SamplingParams(max_new_tokens=30, temperature=0.0))
    b = eng.add_request([4, 5, 6], SamplingParams(max_new_tokens=30, temperature=0.0))
    eng.step()
    eng.step()
    free_before = len(eng.cache.free)
    assert eng.cancel(a.rid) and a.finished and a.finish_reason == "cancelled"
    assert len(eng.cache.free) == free_before + 3                   # 33 tokens = 3 pages came back
    assert not eng.cancel(a.rid)
    n = len(a.generated)
    while eng.has_work():
        eng.step()
    assert len(a.generated) == n and len(b.generated) == 30
    assert len(eng.cache.free) == eng.cache.num_pages


def test_continuous_batching_admits_when_pages_free_up():
    cfg, model = _model()
    eng = ServingEngine(model, device="cpu", dtype=torch.float32, max_batch=8, num_pages=6, max_ctx=64)
    prompts = [[1, 2, 3, 4, 5]] * 4                                 # each needs 2 pages (5 + 20 tokens)
    reqs = [eng.add_request(p, SamplingParams(max_new_tokens=20, temperature=0.0)) for p in prompts]
    eng.step()
    assert len(eng.running) == 3 and len(eng.waiting) == 1          # 6 pages hold three requests
    while eng.has_work():
        eng.step()
    assert all(r.finished and len(r.generated) == 20 for r in reqs)
    assert reqs[0].generated == reqs[3].generated                    # same prompt, greedy


def test_sampler_order_and_limits():
    logits = torch.tensor([[0.0, 1.0, 2.0, 3.0, -1.0]])
    r = Request(0, [3], SamplingParams(temperature=0.0, repetition_penalty=2.0))
    from kotodama_b200.ops import get_ops
    ops = get_ops("cpu")
    assert int(sample_tokens(logits.clone(), [r], ops)[0]) == 3      # token 3 is in the prompt only: not penalised
    r.generated.append(3)
    assert int(sample_tokens(logits.clone(), [r], ops)[0]) == 2      # once generated it is: 3/2 < 2
    r2 = Request(1, [0], SamplingParams(temperature=1.0, top_k=1))
    assert int(sample_tokens(logits.clone(), [r2], ops)[0]) == 3
    draws = set()
    for seed in range(50):
        r3 = Request(2, [0], SamplingParams(temperature=1.0, top_k=0, top_p=0.5, seed=seed))
        draws.add(int(sample_tokens(logits.clone(), [r3], ops)[0]))
    assert draws <= {3}                                              # p(3)=0.64 alone exceeds 0.5
    # the multinomial draw follows the softmax: 4000 seeded draws of a 3-way distribution
    lg = torch.log(torch.tensor([[0.2, 0.5, 0.3]]))
    counts = [0, 0, 0]
    for seed in range(4000):
        counts[int(sample_tokens(lg, [Request(3, [0], SamplingParams(temperature=1.0, top_k=0, seed=seed))], ops)[0])] += 1
    assert abs(counts[0] / 4000 - 0.2) < 0.03 and abs(counts[1] / 4000 - 0.5) < 0.03
    # same seed and draw counter -> same token; the counter is the number of tokens generated so far
    a = Request(4, [0], SamplingParams(temperature=1.0, top_k=0, seed=7))
    b = Request(5, [0], SamplingParams(temperature=1.0, top_k=0, seed=7))
    big = torch.randn(1, 500, generator=torch.Generator().manual_seed(1)) * 3
    assert int(sample_tokens(big, [a], ops)[0]) == int(sample_tokens(big, [b], ops)[0])


def test_page_allocator():
    cfg, _ = _model()
    c = PagedKVCache(cfg, 4, torch.device("cpu"), torch.float32)
    a = c.allocate(3)
    assert len(set(a)) == 3 and not c.can_allocate(2)
    c.release(a)
    assert c.can_allocate(4) and c.pages_for(17) == 2
