"""Parity against the reference's own code (the unmodified LuxiaSL/kotodama package installed
under ``baseline/_ref``), run on CPU in fp32/fp64: state-dict keys and order, loss and every
parameter gradient of ``LuxiaBaseModel`` vs ``KotodamaModel`` (uniform and explicit AttnRes
boundaries, and without AttnRes), ``newton_schulz_orthogonalize`` for the three coefficient
presets, the ``HybridScheduler`` multipliers, one step of the hybrid optimizer, and checkpoints
written by either side loaded by the other.  Skipped when the reference is not installed."""
import importlib
import os
import sys
import types

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")

pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "model")), reason="reference not installed")


@pytest.fixture(scope="module")
def ref():
    """The reference package importable as ``src`` (its modules import ``src.training...``)."""
    if "src" not in sys.modules:
        pkg = types.ModuleType("src")
        pkg.__path__ = [REF]
        sys.modules["src"] = pkg
    ns = types.SimpleNamespace()
    ns.llama = importlib.import_module("src.model.llama")
    ns.muon = importlib.import_module("src.training.muon")
    ns.ckpt = importlib.import_module("src.training.checkpoint")
    return ns


def _cfg_kwargs(attn_res=True, boundaries=None, layers=4):
    return dict(hidden_size=64, num_layers=layers, num_attention_heads=4, num_kv_heads=2, head_dim=16,
                intermediate_size=96, vocab_size=211, max_position_embeddings=64, z_loss_weight=1e-3,
                attn_res=attn_res, attn_res_n_blocks=2, attn_res_boundaries=boundaries)


def _pair(ref, dtype=torch.float64, **kw):
    from kotodama_b200.config import ModelConfig
    from kotodama_b200.models.llama import KotodamaModel
    torch.manual_seed(0)
    theirs = ref.llama.LuxiaBaseModel(ref.llama.LuxiaModelConfig(attn_impl="sdpa", **_cfg_kwargs(**kw))).to(dtype)
    g = torch.Generator().manual_seed(3)
    with torch.no_grad():                      # zero-init pseudo-queries would hide the routing path
        for n, p in theirs.named_parameters():
            if "query" in n:
                p.copy_(torch.randn(p.shape, generator=g, dtype=dtype) * 0.3)
            elif p.ndim == 1:
                p.copy_(1 + 0.1 * torch.randn(p.shape, generator=g, dtype=dtype))
    ours = KotodamaModel(ModelConfig(**_cfg_kwargs(**kw))).to(dtype)
    return theirs, ours


@pytest.mark.parametrize("kw", [dict(), dict(boundaries=[0, 1, 3]), dict(boundaries=[1, 2]), dict(attn_res=False),
                                dict(layers=7, boundaries=[0, 2, 5])])
def test_state_dict_loss_and_gradients_match_the_reference_model(ref, kw):
    theirs, ours = _pair(ref, **kw)
    sd = theirs.state_dict()
    assert list(sd.keys()) == list(ours.state_dict().keys())
    assert [n for n, _ in theirs.named_parameters()] == [n for n, _ in ours.named_parameters()]
    ours.load_state_dict(sd, strict=True)
    ids = torch.randint(0, 211, (3, 24), generator=torch.Generator().manual_seed(1))
    a, b = theirs(ids, labels=ids), ours(ids, labels=ids)
    assert torch.allclose(a["loss"], b["loss"], rtol=1e-10) and torch.allclose(a["z_loss"], b["z_loss"], rtol=1e-10)
    a["loss"].backward()
    b["loss"].backward()
    for (n, p), (_, q) in zip(theirs.named_parameters(), ours.named_parameters()):
        gp = p.grad if p.grad is not None else torch.zeros_like(p)
        gq = q.grad if q.grad is not None else torch.zeros_like(q)
        assert torch.allclose(gp, gq, rtol=1e-8, atol=1e-11), n
    # the hand-scheduled executor (blocked AttnRes schedule included) lands on the same gradients
    from kotodama_b200.engine import TrainEngine
    eng = TrainEngine(ours, device="cpu", dtype=torch.float64)
    loss, _ = eng.forward_backward(ids)
    assert torch.allclose(loss, a["loss"], rtol=1e-9)
    for (n, p), (_, q) in zip(theirs.named_parameters(), ours.named_parameters()):
        gp = p.grad if p.grad is not None else torch.zeros_like(p)
        assert torch.allclose(gp, q.grad, rtol=1e-7, atol=1e-10), n


def test_logits_and_kv_cache_forward_match(ref):
    theirs, ours = _pair(ref, dtype=torch.float32)
    ours.load_state_dict(theirs.state_dict())
    theirs.eval(); ours.eval()
    ids = torch.randint(0, 211, (2, 20), generator=torch.Generator().manual_seed(2))
    with torch.no_grad():
        a = theirs(ids, use_cache=True)
        b = ours(ids, use_cache=True)
        assert torch.allclose(a["logits"], b["logits"], rtol=1e-4, atol=1e-5)
        nxt = a["logits"][:, -1].argmax(-1, keepdim=True)
        a2 = theirs(nxt, past_kv=a["past_kv"], use_cache=True)
        b2 = ours(nxt, past_kv=b["past_kv"], use_cache=True)
        assert torch.allclose(a2["logits"], b2["logits"], rtol=1e-4, atol=1e-5)


@pytest.mark.parametrize("preset", [None, "original", "gram_ns", "polar_express"])
@pytest.mark.parametrize("shape", [(48, 32), (32, 48), (40, 40)])
def test_newton_schulz_matches(ref, preset, shape):
    from kotodama_b200.optim.muon import newton_schulz_orthogonalize
    M = torch.randn(*shape, generator=torch.Generator().manual_seed(4))
    a = ref.muon.newton_schulz_orthogonalize(M, 5, preset)
    b = newton_schulz_orthogonalize(M, 5, preset)
    # both iterate in fp16 on CPU: same arithmetic, same order
    assert torch.allclose(a.float(), b.float(), rtol=2e-2, atol=2e-3)
    assert (a.float() - b.float()).norm() / a.float().norm() < 5e-3


@pytest.mark.parametrize("decay", ["sqrt", "linear", "cosine"])
def test_scheduler_multipliers_match(ref, decay):
    from kotodama_b200.optim.muon import HybridScheduler, build_hybrid_optimizer
    theirs, ours = _pair(ref, dtype=torch.float32)
    ta = ref.muon.build_hybrid_optimizer(theirs)
    oa = build_hybrid_optimizer(ours)
    st = ref.muon.HybridScheduler(*ta, warmup_steps=7, total_steps=50, decay_start_pct=0.8, decay_type=decay)
    so = HybridScheduler(*oa, warmup_steps=7, total_steps=50, decay_start_pct=0.8, decay_type=decay)
    for step in range(50):
        st.step(step)
        so.step(step)
        # the reference evaluates the cosine in fp32 (torch.cos of a float32 tensor)
        assert st.get_last_lr() == pytest.approx(so.get_last_lr(), rel=1e-6 if decay == "cosine" else 1e-12), step


def test_hybrid_optimizer_step_and_parameter_split_match(ref):
    from kotodama_b200.optim.muon import build_hybrid_optimizer
    theirs, ours = _pair(ref, dtype=torch.float32)
    ours.load_state_dict(theirs.state_dict())
    tm, ta = ref.muon.build_hybrid_optimizer(theirs)
    om, oa = build_hybrid_optimizer(ours)
    assert [len(g["params"]) for g in tm.param_groups] == [len(g["params"]) for g in om.param_groups]
    assert sum(len(g["params"]) for g in ta.param_groups) == sum(len(g["params"]) for g in oa.param_groups)
    ids = torch.randint(0, 211, (2, 16), generator=torch.Generator().manual_seed(5))
    start = {n: p.detach().clone() for n, p in theirs.named_parameters()}
    for model, opts in ((theirs, (tm, ta)), (ours, (om, oa))):
        for _ in range(2):
            model(ids, labels=ids)["loss"].backward()
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            for o in opts:
                o.step()
            for o in opts:
                o.zero_grad(set_to_none=True)
    # Newton-Schulz runs in fp16 on both sides (the reference batches same-shape matrices, which changes
    # the rounding), so the updates are compared as a whole: direction and size within a few percent
    for (n, p), (_, q) in zip(theirs.named_parameters(), ours.named_parameters()):
        da, db = p.detach() - start[n], q.detach() - start[n]
        if da.norm() == 0:
            assert db.norm() == 0, n
            continue
        assert (da - db).norm() / da.norm() < 0.05, (n, float((da - db).norm() / da.norm()))


def test_checkpoints_cross_load(ref, tmp_path):
    """A checkpoint written by the reference's manager loads into this framework and back."""
    from kotodama_b200.ckpt.manager import CheckpointManager
    from kotodama_b200.optim.muon import HybridScheduler, build_hybrid_optimizer
    theirs, ours = _pair(ref, dtype=torch.float32)
    tm, ta = ref.muon.build_hybrid_optimizer(theirs)
    om, oa = build_hybrid_optimizer(ours)
    ids = torch.randint(0, 211, (2, 16), generator=torch.Generator().manual_seed(6))
    theirs(ids, labels=ids)["loss"].backward()
    tm.step(); ta.step()
    ts = ref.muon.HybridScheduler(tm, ta, warmup_steps=3, total_steps=20)
    ts.step(5)
    d1 = tmp_path / "theirs"
    ref.ckpt.CheckpointManager(str(d1), rank=0).save(5, theirs, tm, ta, ts, tokens_consumed=1234)
    state = CheckpointManager(str(d1), rank=0).load_latest(ours, om, oa, torch.device("cpu"))
    assert state["step"] == 5 and state["tokens_consumed"] == 1234
    for (n, p), (_, q) in zip(theirs.named_parameters(), ours.named_parameters()):
        assert torch.equal(p, q), n
    # and the other way round
    d2 = tmp_path / "ours"
    so = HybridScheduler(om, oa, warmup_steps=3, total_steps=20)
    so.step(5)
    CheckpointManager(str(d2), rank=0).save(6, ours, om, oa, so, 4321)
    fresh = ref.llama.LuxiaBaseModel(ref.llama.LuxiaModelConfig(attn_impl="sdpa", **_cfg_kwargs()))
    fm, fa = ref.muon.build_hybrid_optimizer(fresh)
    state = ref.ckpt.CheckpointManager(str(d2), rank=0).load_latest(fresh, fm, fa, torch.device("cpu"))
    assert state["step"] == 6 and state["tokens_consumed"] == 4321
    for (n, p), (_, q) in zip(fresh.named_parameters(), ours.named_parameters()):
        assert torch.equal(p, q), n


# ------------------------------------------------------------------------------ monitoring, NCA, metrics
def test_geometric_metric_functions_match(ref):
    """RankMe, stable rank, anisotropy, dead units, attention entropy, the spectrum's power-law exponent and the TwoNN
    dimension on the same tensors (the sampled ones - anisotropy and TwoNN draw subsets - under the same seed)."""
    theirs = importlib.import_module("src.monitoring.geometric")
    from kotodama_b200.monitor import geometric as ours
    g = torch.Generator().manual_seed(0)
    H = torch.randn(300, 48, generator=g) @ torch.diag(torch.linspace(2.0, 0.05, 48))
    W = torch.randn(96, 64, generator=g) @ torch.diag(torch.logspace(0, -2, 64))
    attn = torch.softmax(torch.randn(2, 4, 16, 16, generator=g) * 2, -1)
    hidden = torch.relu(torch.randn(4, 16, 128, generator=g))            # [batch, seq, hidden]
    hidden[..., :13] = 0.0
    assert ours.rankme(H) == pytest.approx(theirs._rankme(H), rel=1e-5)
    assert ours.stable_rank(W) == pytest.approx(theirs._stable_rank(W), rel=1e-5)
    assert ours.dead_unit_fraction(hidden) == pytest.approx(theirs._dead_unit_fraction(hidden), abs=1e-9)
    m0, s0 = theirs._attention_entropy_stats(attn)
    m1, s1 = ours.attention_entropy_stats(attn)
    assert m1 == pytest.approx(m0, rel=1e-5) and s1 == pytest.approx(s0, rel=1e-4)
    torch.manual_seed(1)
    a0 = theirs._anisotropy(H, max_samples=128)
    torch.manual_seed(1)
    a1 = ours.anisotropy(H, max_samples=128)
    assert a1 == pytest.approx(a0, rel=1e-4, abs=1e-6)
    al0, al1 = theirs._weightwatcher_alpha(W), ours.spectrum_alpha(W)
    assert (al0 is None) == (al1 is None) and (al0 is None or al1 == pytest.approx(al0, rel=0.05))
    # a 5-dimensional cloud embedded in 48 dimensions: both estimators land near 5 and near each other
    X = torch.randn(600, 5, generator=g) @ torch.randn(5, 48, generator=g)
    torch.manual_seed(2)
    d0 = theirs._twonn_id(X)
    torch.manual_seed(2)
    d1 = ours.twonn_id(X)
    assert d0 is not None and d1 is not None and abs(d1 - d0) / d0 < 0.1 and 3.5 < d1 < 6.5


def test_nca_tokenisation_and_complexity_match(ref):
    import numpy as np
    theirs = importlib.import_module("src.nca.generator")
    from kotodama_b200.nca import generator as ours
    ct, co = theirs.NCAConfig(grid_size=16, num_steps=6), ours.NCAConfig(grid_size=16, num_steps=6)
    for prop in ("vocab_size", "patches_per_frame", "tokens_per_frame", "tokens_per_timestep", "tokens_per_trajectory"):
        assert getattr(ct, prop) == getattr(co, prop), prop
    traj = torch.randint(0, ct.d_state, (3, 6, ct.n_groups, 16, 16), generator=torch.Generator().manual_seed(0))
    a, b = theirs.tokenize_trajectory(traj, ct.d_state, ct.patch_size), ours.tokenize_trajectory(traj, co.d_state, co.patch_size)
    assert np.array_equal(np.asarray(a).ravel(), np.asarray(b).ravel())
    for toks in (np.asarray(a).ravel(), np.zeros(5000, dtype=np.uint16), np.random.default_rng(0).integers(0, 10000, 5000).astype(np.uint16)):
        assert ours.compute_gzip_complexity(toks) == pytest.approx(theirs.compute_gzip_complexity(toks), rel=1e-9)


def test_metrics_files_and_endpoint_summaries_match(ref, tmp_path):
    import json
    theirs_io = importlib.import_module("src.eval.metrics_io")
    theirs_ra = importlib.import_module("src.eval.run_analysis")
    from kotodama_b200.eval import core as ours_io
    from kotodama_b200.eval import run_analysis as ours_ra
    path = tmp_path / "metrics.jsonl"
    with open(path, "w") as fh:
        for s in range(0, 3000, 10):
            fh.write(json.dumps({"step": s, "timestamp": 1.0, "train/loss": 6.0 * 0.999 ** s + 2.0, "train/perplexity": 50.0,
                                 "perf/tokens_per_sec": 1000.0 + s, "data/tokens_consumed_B": s * 1e-4}) + "\n")
            if s % 500 == 0:
                fh.write(json.dumps({"step": s, "geo/rankme_last": 60.0 - 0.02 * s + 1e-5 * s * s, "geo/ww_alpha_mean": 3.0 - s * 1e-4,
                                     "geo/ww_alpha_healthy_frac": 0.8, "geo/twonn_id/layer_3": 20.0 + s * 1e-3,
                                     "geo/layer_0/stable_rank_q_proj": 10.0 + s * 1e-3, "geo/layer_0/anisotropy": 0.3}) + "\n")
        fh.write("{broken\n")
    a, b = theirs_io.load_metrics(path), ours_io.load_metrics(path)
    assert a == b
    assert theirs_io.extract_series(a, "geo/rankme_last") == ours_io.extract_series(b, "geo/rankme_last")
    assert theirs_io.get_nearest_step(a, 1234) == ours_io.get_nearest_step(b, 1234)
    assert theirs_io.extract_keys_matching(a, "geo/layer_0/") == ours_io.extract_keys_matching(b, "geo/layer_0/")
    assert theirs_io.get_value(a, 500, "geo/anisotropy") == ours_io.get_value(b, 500, "geo/anisotropy")
    st, so = theirs_ra.endpoint_summary(a), ours_ra.endpoint_summary(b)
    for k, v in st.items():                       # every figure the reference reports, to rounding
        assert k in so, k
        if isinstance(v, float):
            assert so[k] == pytest.approx(v, rel=1e-9), k
        else:
            assert so[k] == v, k


def test_analysis_forward_and_perplexity_match(ref, tmp_path):
    """The analysis forward pass (states after every layer, attention probabilities) and the held-out perplexity
    against the reference's ``src/eval`` on the same weights.  Without AttnRes: the reference's analysis copy of the
    AttnRes forward deliberately is not the yardstick (it omits the reset of the partial sum at block boundaries that
    its own model performs; the model-level test above pins the AttnRes numerics instead)."""
    import warnings

    import numpy as np
    theirs_fw = importlib.import_module("src.eval.forward")
    theirs_ppl = importlib.import_module("src.eval.perplexity")
    from kotodama_b200.eval import compute_perplexity, forward_with_states
    theirs, ours = _pair(ref, dtype=torch.float32, attn_res=False)
    ours.load_state_dict(theirs.state_dict())
    theirs.eval(), ours.eval()
    ids = torch.randint(0, 211, (2, 24), generator=torch.Generator().manual_seed(5))
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")                      # "cuda autocast requested but CUDA is not available"
        a = theirs_fw.forward_with_states(theirs, ids, capture_attention=True, attention_layers=[0, 3])
        b = forward_with_states(ours, ids, attention_layers=[0, 3])
        assert len(a.states) == len(b.states) == 5
        for x, y in zip(a.states[:-1], b.states[:-1]):       # the last entry is the normed output here, the raw state there
            assert torch.allclose(x.float(), y.float(), atol=2e-5, rtol=1e-4)
        for l in (0, 3):
            w = a.attention_weights[l]
            w = torch.as_tensor(w)
            got = b.attention[l]
            assert torch.allclose(w.reshape(got.shape[1:]).float(), got[0].float(), atol=2e-5)      # the reference keeps sequence 0
        toks = np.random.default_rng(0).integers(0, 211, 40 * 32).astype("<u2")
        toks.tofile(tmp_path / "eval.bin")
        pa = theirs_ppl.compute_perplexity(theirs, tmp_path / "eval.bin", seq_len=32, batch_size=4, max_seqs=40, device="cpu")
        pb = compute_perplexity(ours, tmp_path / "eval.bin", seq_len=32, batch_size=4, max_tokens=40 * 32)
    assert pb["loss"] == pytest.approx(pa["loss"], rel=1e-5) and pb["perplexity"] == pytest.approx(pa["perplexity"], rel=1e-4)
    assert int(pb["tokens"]) == int(pa["n_tokens"])


def test_sampler_distribution_matches_the_reference_server(ref, monkeypatch):
    """The serving sampler (repetition penalty -> temperature -> top-k -> top-p -> multinomial) against the reference
    server's ``sample_next_token``: the reference's filtered probabilities are captured at its ``torch.multinomial``
    call; ours are measured by sweeping the sampler's uniform draw over a fine grid (inverse-CDF sampling cuts [0, 1)
    into intervals whose lengths are the probabilities)."""
    import importlib.util
    serve_py = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")), "serve.py")
    if not os.path.isfile(serve_py):
        pytest.skip("the reference's serve.py is not on this machine")
    spec = importlib.util.spec_from_file_location("reference_serve", serve_py)
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)
    from kotodama_b200.ops.reference import TorchOps
    ours = TorchOps()
    V, N = 40, 4000
    g = torch.Generator().manual_seed(0)
    seen_ids = [3, 7, 7, 11, 30]
    for temperature, top_k, top_p, rp in [(0.7, 0, 0.0, 1.0), (1.3, 8, 0.0, 1.0), (0.9, 0, 0.8, 1.0), (1.0, 12, 0.6, 1.3), (0.5, 5, 0.95, 1.8)]:
        logits = torch.randn(V, generator=g) * 2.5
        captured = {}

        def fake_multinomial(probs, num_samples=1, **kw):
            captured["p"] = probs.detach().clone()
            return probs.argmax().reshape(1)
        monkeypatch.setattr(torch, "multinomial", fake_multinomial)
        theirs.sample_next_token(logits.clone(), temperature, top_k, top_p, rp, list(seen_ids))
        monkeypatch.undo()
        want = captured["p"].double()
        words = torch.zeros(1, (V + 31) // 32, dtype=torch.int32)
        for t in set(seen_ids):
            words[0, t >> 5] |= 1 << (t & 31)
        counts = torch.zeros(V, dtype=torch.double)
        for i in range(N):
            ours.sample_uniform = lambda seed, counter, u=(i + 0.5) / N: u
            tok = ours.sample(logits.clone()[None], [temperature], [top_k], [top_p], [rp], [0], [0], words.clone(), [0])
            counts[int(tok)] += 1
        got = counts / N
        assert not bool(((got > 0) & (want == 0)).any())               # nothing outside the reference's support
        assert bool((got[want > 2.0 / N] > 0).all())                   # everything inside it that the grid can resolve
        assert float((got - want).abs().max()) < 2.5 / N, (temperature, top_k, top_p, rp)
    # greedy: same token, penalty included
    logits = torch.randn(V, generator=g)
    a = theirs.sample_next_token(logits.clone(), 0.0, 0, 0.0, 1.5, list(seen_ids))
    b = ours.sample(logits.clone()[None], [0.0], [0], [0.0], [1.5], [0], [0], words.clone(), [0])
    assert a == int(b)


def test_paged_serving_engine_generates_what_the_reference_server_generates(ref):
    """End to end on the same weights (fp32, CPU): the reference server's ``generate`` (contiguous KV cache, one request)
    against this package's engine (paged cache, continuous batching, several requests at once), greedy with and without
    a repetition penalty, AttnRes with explicit boundaries."""
    import importlib.util
    serve_py = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")), "serve.py")
    if not os.path.isfile(serve_py):
        pytest.skip("the reference's serve.py is not on this machine")
    spec = importlib.util.spec_from_file_location("reference_serve", serve_py)
    theirs_srv = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs_srv)
    from kotodama_b200.serve.engine import SamplingParams, ServingEngine
    theirs, ours = _pair(ref, dtype=torch.float32, boundaries=[0, 1, 3])
    ours.load_state_dict(theirs.state_dict())
    theirs.eval(), ours.eval()

    class Tok:                                   # ids in, ids out: the text is the id list
        eos_token_id = -1

        def encode(self, prompt, return_tensors=None):
            return torch.tensor([[int(t) for t in prompt.split()]])

        def decode(self, ids, skip_special_tokens=True):
            return " ".join(str(int(i)) for i in ids)
    prompts = [[5, 17, 3, 99, 42], [7] * 11, [200, 1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 13, 14, 15, 16, 17]]
    eng = ServingEngine(ours, device="cpu", dtype=torch.float32, max_batch=4, max_ctx=64)
    seen = {}
    for rp in (1.0, 2.0):
        want = []
        for p in prompts:
            req = theirs_srv.GenerateRequest(prompt=" ".join(map(str, p)), max_new_tokens=14, temperature=0.0, top_k=0, top_p=0.0,
                                             repetition_penalty=rp)
            want.append([int(t) for t in theirs_srv.generate(theirs, Tok(), req).text.split()])
        got = eng.generate(prompts, SamplingParams(max_new_tokens=14, temperature=0.0, repetition_penalty=rp))
        assert got == want, rp
        seen[rp] = want
    assert seen[1.0] != seen[2.0]                # the penalty changes at least one continuation, so the second case means something


def test_executor_training_steps_track_the_reference_loop(ref):
    """Several optimizer steps of the hand-scheduled executor (own backward schedule, fused clip + Muon + AdamW) against
    the reference's loop (autograd, ``clip_grad_norm_``, its Muon and AdamW, its scheduler stepped after the
    optimizers) on the same weights and the same fixed batch, fp32 on the CPU.  Both sides run Newton-Schulz in half
    precision with different batching, so the trajectories agree closely, not bit for bit."""
    from kotodama_b200.engine import TrainEngine
    from kotodama_b200.optim.muon import HybridScheduler
    theirs, ours = _pair(ref, dtype=torch.float32, boundaries=[0, 1, 3])
    ours.load_state_dict(theirs.state_dict())
    tm, ta = ref.muon.build_hybrid_optimizer(theirs, muon_lr=0.02, adamw_lr=3e-3)
    ts = ref.muon.HybridScheduler(tm, ta, warmup_steps=2, total_steps=8)
    eng = TrainEngine(ours, device="cpu", dtype=torch.float32, muon_lr=0.02, adamw_lr=3e-3, gradient_clip=1.0)
    os_ = HybridScheduler(eng.muon_opt, eng.adamw_opt, warmup_steps=2, total_steps=8)
    ids = torch.randint(0, 211, (3, 32), generator=torch.Generator().manual_seed(9))
    la, lb, na, nb = [], [], [], []
    for step in range(8):
        out = theirs(ids, labels=ids)
        out["loss"].backward()
        na.append(float(torch.nn.utils.clip_grad_norm_(theirs.parameters(), 1.0)))
        tm.step(); ta.step()
        tm.zero_grad(set_to_none=True); ta.zero_grad(set_to_none=True)
        ts.step(step)
        la.append(float(out["loss"].detach()))
        if step == 0:
            za = float(out["z_loss"].detach())
        r = eng.train_step([ids])
        os_.step(step)
        if step == 0:
            zb = float(r["z_loss"])
        lb.append(float(r["loss"]))
        nb.append(float(r["grad_norm"]))
    # step 0: identical weights -> the same loss (z-loss included on both sides), z-loss and gradient norm
    assert lb[0] == pytest.approx(la[0], rel=1e-5) and zb == pytest.approx(za, rel=1e-4)
    assert nb[0] == pytest.approx(na[0], rel=1e-3)
    for a, b in zip(la, lb):
        assert abs(a - b) < 0.03 * max(abs(a), 1.0), (la, lb)
    assert la[-1] < la[0] - 0.3 and lb[-1] < lb[0] - 0.3


@pytest.mark.parametrize("attn_res", [True, False])
def test_geometric_monitor_series_match(ref, attn_res):
    """Both monitors on the same weights and probe batch: the same metric keys (layer samples included) and, with
    AttnRes, the same values for every tier-1 series and the TwoNN dimensions.  Without AttnRes the attention entropy is
    left out of the value comparison: the reference's plain path feeds a layer's output back into that layer's attention,
    this package records the probabilities the layer really used."""
    import warnings
    theirs_geo = importlib.import_module("src.monitoring.geometric")
    from kotodama_b200.monitor import geometric as ours_geo
    theirs, ours = _pair(ref, dtype=torch.float32, attn_res=attn_res, boundaries=[0, 1, 3] if attn_res else None)
    ours.load_state_dict(theirs.state_dict())
    theirs.eval(), ours.eval()
    ids = torch.randint(0, 211, (6, 32), generator=torch.Generator().manual_seed(1))
    mt = theirs_geo.GeometricMonitor(theirs, theirs_geo.MonitorConfig(device="cpu"))
    mo = ours_geo.GeometricMonitor(ours, ours_geo.MonitorConfig(device="cpu"))
    assert mt.config.tier1_sample_layers == mo.config.tier1_sample_layers
    assert mt.config.tier2_twonn_layers == mo.config.tier2_twonn_layers
    mt.set_probe_batch(ids)
    mo.set_probe_batch(ids)
    with warnings.catch_warnings():
        warnings.simplefilter("ignore")
        torch.manual_seed(0)
        a1 = mt.tier1(100)
        torch.manual_seed(0)
        b1 = mo.tier1(100)
        torch.manual_seed(0)
        a2 = mt.tier2(100)
        torch.manual_seed(0)
        b2 = mo.tier2(100)
    assert set(a1) == set(b1)
    assert set(a2) <= set(b2)                       # this package also reports k / v / up and the by-type means
    for k, v in a1.items():
        if "time" in k or (not attn_res and "attn_entropy" in k):
            continue
        assert b1[k] == pytest.approx(v, rel=1e-3, abs=1e-5), k
    for k, v in a2.items():
        if k.startswith("geo/twonn_id/"):
            assert b2[k] == pytest.approx(v, rel=1e-3), k


def test_metric_files_written_by_both_loggers_are_interchangeable(ref, tmp_path):
    """Twelve training steps and two geometric records through the reference's logger and this package's: the same
    JSONL records (keys and values; the loss slope appears from the tenth step on both sides), so either analysis stack
    reads either run."""
    import json
    theirs_log = importlib.import_module("src.monitoring.wandb_callback")
    from kotodama_b200.eval import load_metrics
    from kotodama_b200.monitor.logger import WandbLogger
    a = theirs_log.WandbLogger(project="p", run_name="r", config={"x": 1}, log_dir=str(tmp_path / "theirs"), enabled=True)
    b = WandbLogger(project="p", run_name="r", config={"x": 1}, log_dir=str(tmp_path / "ours"), enabled=True, use_wandb=False)
    for lg in (a, b):
        for step in range(12):
            lg.log_step(step, loss=5.0 - 0.1 * step, z_loss=1e-3, grad_norm=1.5, muon_lr=0.02, adamw_lr=6e-4, tokens_per_sec=1000.0 + step,
                        tokens_consumed=4096 * (step + 1), gpu_mem_gb=12.5, step_time_s=0.5, iters_per_sec=2.0)
            if step in (5, 10):
                lg.log_geo(step, {"geo/rankme_last": 40.0 + step, "geo/layer_0/anisotropy": 0.1})
            lg.commit(step)
        lg.finish()

    def records(d, name):
        out = []
        for line in open(d / name):
            r = json.loads(line)
            r.pop("timestamp", None)
            r.pop("_timestamp", None)
            out.append(r)
        return out
    for name in ("metrics.jsonl", "geo_metrics.jsonl"):
        ra, rb = records(tmp_path / "theirs", name), records(tmp_path / "ours", name)
        assert len(ra) == len(rb) and len(ra) > 0, name
        for x, y in zip(ra, rb):
            assert set(x) == set(y), (name, set(x) ^ set(y))
            for k in x:
                assert y[k] == pytest.approx(x[k], rel=1e-9, abs=1e-12) if isinstance(x[k], float) else y[k] == x[k], (name, k)
    assert load_metrics(tmp_path / "theirs" / "metrics.jsonl") == load_metrics(tmp_path / "ours" / "metrics.jsonl")


def test_nca_rule_network_and_update_match(ref):
    """The cellular-automaton rule network with the reference's weights: perception convolution with wrap-around
    padding, 1 x 1 hidden layers, output logits per group - the same logits for the same grid."""
    theirs = importlib.import_module("src.nca.generator")
    from kotodama_b200.nca import generator as ours
    d, G, K, Hd, nh, S = 10, 4, 3, 32, 2, 12
    torch.manual_seed(0)
    a = theirs.NCARule(d, G, K, Hd, nh)
    b = ours.NCARule(d, G, K, Hd, nh)
    sd = a.state_dict()
    names = ["perception"] + [k.rsplit(".", 1)[0] for k in sd if k.startswith("hidden.") and k.endswith(".weight")] + ["output"]
    with torch.no_grad():
        for i, n in enumerate(names):
            b.weights[i].copy_(sd[f"{n}.weight"])
            b.biases[i].copy_(sd[f"{n}.bias"])
    state = torch.randint(0, d, (2, G, S, S), generator=torch.Generator().manual_seed(1))
    onehot = torch.nn.functional.one_hot(state, d).permute(0, 1, 4, 2, 3).reshape(2, G * d, S, S).float()
    la, lb = a(onehot), b(onehot)
    assert la.shape == lb.shape and torch.allclose(la, lb, atol=1e-5)
    # the borders matter: a cell on the edge sees the opposite edge
    assert not torch.allclose(la[..., 0, :], la[..., S // 2, :])


@pytest.mark.parametrize("kw", [dict(), dict(attn_res=False), dict(boundaries=[0, 1, 3])])
def test_initialisation_and_reinitialisation_draw_the_same_weights(ref, kw):
    """Under one seed both models are initialised to the same tensors (scheme, standard deviations and the order in
    which parameters are drawn), and ``reinit_mlps`` / ``reinit_embeddings`` (the NCA -> language transition) redraw
    the same ones."""
    from kotodama_b200.config import ModelConfig
    from kotodama_b200.models.llama import KotodamaModel
    torch.manual_seed(11)
    theirs = ref.llama.LuxiaBaseModel(ref.llama.LuxiaModelConfig(attn_impl="sdpa", **_cfg_kwargs(**kw)))
    torch.manual_seed(11)
    ours = KotodamaModel(ModelConfig(**_cfg_kwargs(**kw)))
    sa, sb = theirs.state_dict(), ours.state_dict()
    assert list(sa) == list(sb)
    for k in sa:
        assert torch.equal(sa[k], sb[k]), k
    torch.manual_seed(12)
    theirs.reinit_mlps()
    theirs.reinit_embeddings(new_vocab_size=300)
    torch.manual_seed(12)
    ours.reinit_mlps()
    ours.reinit_embeddings(new_vocab_size=300)
    sa, sb = theirs.state_dict(), ours.state_dict()
    assert sb["embed_tokens.weight"].shape == (300, 64) and ours.config.vocab_size == 300
    for k in sa:
        assert torch.equal(sa[k], sb[k]), k


def test_asynchronous_checkpoints_cross_load(ref, tmp_path):
    """The background-writer managers of both code bases (host clone, staging directory, persist, rotation): a file
    written by either loads into the other with the same step, token count, parameters and optimizer moments, and both
    keep the same number of files."""
    from kotodama_b200.ckpt.manager import AsyncCheckpointManager
    from kotodama_b200.optim.muon import HybridScheduler, build_hybrid_optimizer
    theirs, ours = _pair(ref, dtype=torch.float32)
    ours.load_state_dict(theirs.state_dict())
    tm, ta = ref.muon.build_hybrid_optimizer(theirs)
    om, oa = build_hybrid_optimizer(ours)
    ids = torch.randint(0, 211, (2, 16), generator=torch.Generator().manual_seed(6))
    for model, opts in ((theirs, (tm, ta)), (ours, (om, oa))):
        model(ids, labels=ids)["loss"].backward()
        for o in opts:
            o.step()
    ts = ref.muon.HybridScheduler(tm, ta, warmup_steps=3, total_steps=50)
    so = HybridScheduler(om, oa, warmup_steps=3, total_steps=50)
    a = ref.ckpt.AsyncCheckpointManager(str(tmp_path / "theirs"), rank=0, keep_last_n=2, shm_dir=str(tmp_path / "shm_a"), compress=False)
    b = AsyncCheckpointManager(str(tmp_path / "ours"), rank=0, keep_last_n=2, shm_dir=str(tmp_path / "shm_b"), compress=False)
    for step in (10, 20, 30):
        ts.step(step)
        so.step(step)
        a.save(step, theirs, tm, ta, ts, tokens_consumed=1000 * step)
        b.save(step, ours, om, oa, so, tokens_consumed=1000 * step)
    a.shutdown()
    b.shutdown()
    fa = sorted(p.name for p in (tmp_path / "theirs").glob("step_*.pt*"))
    fb = sorted(p.name for p in (tmp_path / "ours").glob("step_*.pt*"))
    assert fa == fb == ["step_00000020.pt", "step_00000030.pt"]
    # theirs -> ours
    fresh = _pair(ref, dtype=torch.float32)[1]
    fm, fa_ = build_hybrid_optimizer(fresh)
    state = AsyncCheckpointManager(str(tmp_path / "theirs"), rank=0, shm_dir=str(tmp_path / "shm_c"), compress=False).load_latest(
        fresh, fm, fa_, torch.device("cpu"))
    assert state["step"] == 30 and state["tokens_consumed"] == 30000
    for (n, p), (_, q) in zip(theirs.named_parameters(), fresh.named_parameters()):
        assert torch.equal(p, q), n
    mom_a = [s["momentum_buffer"] for s in tm.state.values() if "momentum_buffer" in s]
    mom_b = [s["momentum_buffer"] for s in fm.state.values() if "momentum_buffer" in s]
    assert len(mom_a) == len(mom_b) > 0 and all(torch.equal(x, y) for x, y in zip(mom_a, mom_b))
    # ours -> theirs
    fresh_t = _pair(ref, dtype=torch.float32)[0]
    gm, ga = ref.muon.build_hybrid_optimizer(fresh_t)
    state = ref.ckpt.AsyncCheckpointManager(str(tmp_path / "ours"), rank=0, shm_dir=str(tmp_path / "shm_d"), compress=False).load_latest(
        fresh_t, gm, ga, torch.device("cpu"))
    assert state["step"] == 30 and state["tokens_consumed"] == 30000
    for (n, p), (_, q) in zip(ours.named_parameters(), fresh_t.named_parameters()):
        assert torch.equal(p, q), n


def _reference_trainer():
    """The reference's train.py as a module (for its parser and pure helpers).  It imports ``src.data.dataset``, a
    module the upstream repository does not contain; the dataset classes of this package stand in for it."""
    import types as _types
    if "src.data.dataset" not in sys.modules:
        data = _types.ModuleType("src.data")
        data.__path__ = []
        ds = _types.ModuleType("src.data.dataset")
        from kotodama_b200.data.dataset import RandomTokenDataset, TokenizedDataset
        ds.RandomTokenDataset, ds.TokenizedDataset = RandomTokenDataset, TokenizedDataset
        sys.modules["src.data"], sys.modules["src.data.dataset"] = data, ds
    return importlib.import_module("src.training.train")


def test_training_flags_defaults_and_batch_ramp_match(ref, monkeypatch, tmp_path):
    """Every flag of the reference's trainer exists here with the same default; a YAML file plus command-line overrides
    resolve to the same values; the batch-size ramp gives the same accumulation count at every step."""
    from kotodama_b200.config import grad_accum_for_step, parse_args
    theirs = _reference_trainer()
    monkeypatch.setattr(sys, "argv", ["train.py"])
    a, b = vars(theirs.parse_args()), vars(parse_args([]))
    assert set(a) <= set(b), sorted(set(a) - set(b))
    assert {k: (a[k], b[k]) for k in a if a[k] != b[k]} == {}
    cfg = tmp_path / "run.yaml"
    cfg.write_text("model_size: 3b\nmicro_batch_size: 4\nmuon_lr: 0.015\nattn_res: true\nattn_res_boundaries: \"0,3,7\"\n"
                   "decay_type: cosine\nsave_every: 123\nwandb: false\nfp8: true\n")
    argv = ["--config", str(cfg), "--micro_batch_size", "2", "--warmup_steps", "77", "--async_checkpoint"]
    monkeypatch.setattr(sys, "argv", ["train.py", *argv])
    a, b = vars(theirs.parse_args()), vars(parse_args(argv))
    assert {k: (a[k], b[k]) for k in a if a[k] != b[k]} == {}
    assert b["micro_batch_size"] == 2 and b["muon_lr"] == 0.015 and b["save_every"] == 123 and b["fp8"] is True
    for total, base, frac, pct in [(1000, 16, 0.25, 0.05), (1000, 16, 1.0, 0.05), (500, 7, 0.1, 0.2), (10, 4, 0.5, 0.0), (40, 3, 0.3, 0.5)]:
        for step in range(0, total, max(total // 50, 1)):
            assert grad_accum_for_step(step, total, base, frac, pct) == theirs._compute_grad_accum_for_step(
                step, total, base, initial_batch_fraction=frac, ramp_pct=pct), (step, total, base, frac, pct)


def test_model_presets_and_gradient_diagnostics_match(ref):
    """The size presets (tiny and the profile-only ones aside) carry the reference's dimensions, the parameter-count
    estimate agrees, and the per-layer attention / MLP gradient norms the trainer logs are the same numbers."""
    from kotodama_b200.config import MODEL_PRESETS, ModelConfig
    from kotodama_b200.train import per_layer_grad_norms
    theirs = _reference_trainer()
    shared = set(theirs.MODEL_CONFIGS) & set(MODEL_PRESETS)
    assert {"full", "3b", "8b", "proxy", "intermediate", "smoke"} <= shared
    for name in shared:
        a, b = theirs.MODEL_CONFIGS[name], MODEL_PRESETS[name]
        assert {k: (a[k], b.get(k)) for k in a if a[k] != b.get(k)} == {}, name
        ca, cb = ref.llama.LuxiaModelConfig(**a), ModelConfig(**b)
        assert ca.param_count() == cb.param_count(), name
    t, o = _pair(ref, dtype=torch.float32, layers=9)
    o.load_state_dict(t.state_dict())
    ids = torch.randint(0, 211, (2, 16), generator=torch.Generator().manual_seed(8))
    t(ids, labels=ids)["loss"].backward()
    o(ids, labels=ids)["loss"].backward()
    ga, gb = theirs._per_layer_grad_norms(t), per_layer_grad_norms(o)
    assert set(ga) == set(gb) and {"grad/layer_0/attn", "grad/layer_4/mlp", "grad/layer_8/attn_mlp_ratio"} <= set(ga)
    for k, v in ga.items():
        assert gb[k] == pytest.approx(v, rel=1e-4), k


def test_concept_geometry_statistics_match_the_reference_script(ref):
    """The structure statistics of the concept-geometry track against the functions of the reference's
    ``scripts/analysis/analyze_concept_geometry.py``: target distance matrices, Spearman Mantel rho (ties included),
    cyclic-neighbour hit rate and ordinal window overlap, on a noisy ring, a noisy line and pure noise."""
    import importlib.util
    import math

    import numpy as np
    script = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")),
                          "scripts", "analysis", "analyze_concept_geometry.py")
    if not os.path.isfile(script):
        pytest.skip("the reference's analysis scripts are not on this machine")
    spec = importlib.util.spec_from_file_location("reference_concepts", script)
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)
    sys.path.insert(0, os.path.join(ROOT, "tools", "analysis"))
    import analyze_concept_geometry as ours
    rng = np.random.default_rng(0)
    n = 12
    ang = np.arange(n) / n * 2 * math.pi
    clouds = {"ring": np.stack([np.cos(ang), np.sin(ang)], 1) @ rng.normal(size=(2, 16)) + rng.normal(size=(n, 16)) * 0.15,
              "line": np.arange(n, dtype=float)[:, None] @ rng.normal(size=(1, 16)) + rng.normal(size=(n, 16)) * 0.8,
              "noise": rng.normal(size=(n, 16))}
    assert np.array_equal(theirs.cyclic_distance_matrix(n), ours.target_dist(n, True))
    assert np.array_equal(theirs.ordinal_distance_matrix(n), ours.target_dist(n, False))
    for name, x in clouds.items():
        d = ours.pdist(x - x.mean(0))
        for cyclic in (True, False):
            tgt = ours.target_dist(n, cyclic)
            rho_t, p_t = theirs.mantel_test(d, tgt, n_perm=300, seed=1)
            got = ours.mantel(d, tgt, 300, np.random.default_rng(1))
            assert got["r"] == pytest.approx(rho_t, abs=1e-9), (name, cyclic)
            assert abs(got["p"] - p_t) < 0.08, (name, cyclic, got["p"], p_t)         # same null, different draws
        for k in (1, 2):
            assert ours.knn_cyclic_hit(d, k) == pytest.approx(theirs.knn_cyclic(d, n, k)), name
        assert ours.knn_ordinal_window(d, 3, 2) == pytest.approx(theirs.knn_ordinal_overlap(d, n, 3, 2)), name
    assert ours.mantel(ours.pdist(clouds["ring"]), ours.target_dist(n, True), 200, np.random.default_rng(2))["p"] < 0.02


def test_text_quality_formulas_match_the_reference_script(ref):
    """The closed-form pieces of the text-quality track (type/token ratios of a sample's head, Yule's K, Honore's R,
    n-grams, slope, entropy) against the reference's ``scripts/analysis/analyze_text_quality.py``.  That script needs
    NLTK for tokenising and tagging; a stand-in module lets it import, and only functions that take word lists are
    compared (this package tokenises with regular expressions instead, so the full metrics differ by design)."""
    import importlib.util
    import types as _types
    script = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")),
                          "scripts", "analysis", "analyze_text_quality.py")
    if not os.path.isfile(script):
        pytest.skip("the reference's analysis scripts are not on this machine")
    added = []
    if "nltk" not in sys.modules:
        try:
            import nltk  # noqa: F401
        except ImportError:
            fake = _types.ModuleType("nltk")
            fake.pos_tag = fake.sent_tokenize = fake.word_tokenize = lambda *a, **k: []
            fake.download = lambda *a, **k: True
            fake.data = _types.SimpleNamespace(find=lambda *a, **k: True)
            tok = _types.ModuleType("nltk.tokenize")
            tok.RegexpTokenizer = lambda *a, **k: None
            sys.modules["nltk"], sys.modules["nltk.tokenize"] = fake, tok
            added = ["nltk", "nltk.tokenize"]
    try:
        spec = importlib.util.spec_from_file_location("reference_text_quality", script)
        theirs = importlib.util.module_from_spec(spec)
        sys.modules["reference_text_quality"] = theirs          # its dataclasses look their module up by name
        spec.loader.exec_module(theirs)
    finally:
        for m in added:
            sys.modules.pop(m, None)
    sys.path.insert(0, os.path.join(ROOT, "tools", "analysis"))
    import analyze_text_quality as ours
    import random
    rnd = random.Random(0)
    vocab = [f"w{i}" for i in range(60)]
    samples = [[rnd.choice(vocab[: 5 + i * 11]) for _ in range(40 + 90 * i)] for i in range(6)] + [["a"] * 30, ["a", "b"], []]
    for ws in samples:
        for window in (50, 100, 200, 500):
            assert ours.head_ttr(ws, window) == pytest.approx(theirs.compute_ttr(ws, window)), (len(ws), window)
        assert ours.yules_k(ws) == pytest.approx(theirs.compute_yules_k(ws)), len(ws)
        assert ours.honores_r(ws) == pytest.approx(theirs.compute_honores_r(ws)), len(ws)
        for n in (1, 3, 5):
            assert ours.ngrams(ws, n) == theirs.get_ngrams(ws, n)
    for ys in ([1.0, 2.0, 4.0, 8.0], [3.0], [], [5.0, 5.0, 5.0], [9.0, 7.0, 2.0, 2.5, 0.1]):
        assert ours.slope(ys) == pytest.approx(theirs.linear_slope(ys))
    for counts in ([1, 1, 1, 1], [10, 1], [7], [3, 0, 5]):
        tot = sum(counts)
        assert ours.entropy(counts) == pytest.approx(theirs.entropy([c / tot for c in counts]))


def _reference_tool(name: str) -> str:
    path = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")), "tools", name)
    if not os.path.isfile(path):
        pytest.skip("the reference's tools are not on this machine")
    return path


def test_training_log_is_read_alike_by_the_reference_log_tool_and_ours(tmp_path):
    """A log written by this package's trainer goes through the reference's ``tools/extract_benchmark_results.py``
    (its ``extract_metrics`` takes the log text) and through ``tools/extract_benchmark_results.py`` here: both see the
    same tokens/s samples and memory figure, i.e. the step line keeps the reference's format."""
    import importlib.util
    import logging
    from kotodama_b200.train import parse_args, train
    spec = importlib.util.spec_from_file_location("reference_extract", _reference_tool("extract_benchmark_results.py"))
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)
    sys.path.insert(0, os.path.join(ROOT, "tools"))
    import extract_benchmark_results as ours
    log = tmp_path / "train.log"
    handler = logging.FileHandler(log)
    handler.setFormatter(logging.Formatter("%(message)s"))
    logging.getLogger("kotodama_b200.train").addHandler(handler)
    try:
        train(parse_args(["--config", os.path.join(ROOT, "configs", "tiny-cpu.yaml"), "--total_steps", "9", "--log_every", "1",
                          "--save_every", "999999", "--checkpoint_dir", str(tmp_path / "ck")]))
    finally:
        logging.getLogger("kotodama_b200.train").removeHandler(handler)
        handler.close()
    text = log.read_text()
    got_theirs = theirs.extract_metrics(text)
    got_ours = ours.summarise(str(log), skip=5)
    import re
    import numpy as np
    samples = [float(v) for v in re.findall(r"tok/s=(\d+\.?\d*)", text)]
    assert len(samples) == 9 and got_ours["lines"] == 9
    assert got_theirs["n_samples"] == 4 and got_theirs["peak_tok_per_sec"] == int(max(samples))
    assert got_theirs["min_tok_per_sec"] == int(min(samples[5:])) and got_theirs["avg_tok_per_sec"] == int(sum(samples[5:]) / 4)
    assert got_ours["tok_s_median"] == pytest.approx(float(np.median(samples[5:])))
    assert got_theirs["peak_gpu_mem_gb"] == got_ours["gpu_mem_gb_max"] == 0.0


def test_trace_summary_matches_the_reference_trace_tool(tmp_path):
    """The same chrome trace through the reference's ``tools/parse_profile.py`` (run as the script it is) and through
    ``tools/parse_profile.py`` here: kernel order, totals, counts and the host-op table agree."""
    import json
    import subprocess
    import numpy as np
    rng = np.random.default_rng(0)
    events = []
    for i in range(200):
        events.append({"cat": "kernel", "name": f"kernel_{int(rng.integers(0, 12))}", "dur": int(rng.integers(1, 5000)), "ts": i})
        events.append({"cat": "cpu_op", "name": f"aten::op_{int(rng.integers(0, 6))}", "dur": int(rng.integers(1, 900)), "ts": i})
    events += [{"cat": "user_annotation", "name": "FORWARD", "dur": 123456, "ts": 0}, {"cat": "kernel", "name": "zero_dur", "dur": 0},
               {"cat": "gpu_memcpy", "name": "Memcpy HtoD", "dur": 77}]
    trace = tmp_path / "t.json"
    trace.write_text(json.dumps({"traceEvents": events}))
    theirs = subprocess.run([sys.executable, _reference_tool("parse_profile.py"), str(trace)], capture_output=True, text=True, check=True).stdout
    sys.path.insert(0, os.path.join(ROOT, "tools"))
    import parse_profile as ours
    rows = ours.parse(str(trace), top=30)
    their_rows = [l.split() for l in theirs.split("-" * 125)[1].split("\nTop 30")[0].strip().splitlines()]
    assert [r[0] for r in their_rows] == [r[0] for r in rows]
    for (name, total_us, count), t in zip(rows, their_rows):
        assert float(t[1]) == pytest.approx(total_us / 1e3, abs=0.051) and int(t[2]) == count
    total_s = sum(r[1] for r in rows) / 1e6
    assert f"Total CUDA kernel time: {total_s:.1f}s" in theirs and f"Unique CUDA kernels: {len(rows)}" in theirs
    host = ours.parse_cpu(str(trace))
    their_host = [l.split() for l in theirs.split("\n" + "-" * 110 + "\n")[1].strip().splitlines()]
    assert [r[0] for r in their_host] == [r[0] for r in host] and host[0][0] == "FORWARD"
    assert all(int(t[2]) == h[2] for t, h in zip(their_host, host))


def test_training_dynamics_figures_match_the_reference_engine(ref):
    """The shared definitions of the run-analysis engine on one noisy 20 000-step run with two planted jumps: slopes in
    centred windows at the landmark steps (all four window sizes), 500-step rolling mean / spread / count, the stability
    score, and the jump detector (step, size, sigma) against ``src/eval/run_analysis.py``."""
    import numpy as np
    theirs = importlib.import_module("src.eval.run_analysis")
    from kotodama_b200.eval import run_analysis as ours
    rng = np.random.default_rng(3)
    data = {}
    for s in range(0, 20001, 10):
        loss = 2.5 + 4.0 * np.exp(-s / 3000.0) + rng.normal(0, 0.02 * (1.0 + 3.0 * np.exp(-s / 2000.0)))
        loss += 0.6 if s == 7000 else 0.0
        loss -= 0.5 if s >= 15000 else 0.0
        data[s] = {"train/loss": float(loss), "geo/rankme_last": float(40 + 0.001 * s + rng.normal(0, 0.3))}
    a = theirs.training_dynamics(data, ["train/loss", "geo/rankme_last"])["metrics"]
    b = ours.training_dynamics(data, ["train/loss", "geo/rankme_last"])
    for key in ("train/loss", "geo/rankme_last"):
        for pct in (10, 25, 50, 75, 90):
            for w in (100, 500, 1000, 5000):
                x, y = a[key]["slopes_at_landmarks"][f"pct_{pct}"][f"w{w}"], b[key]["slopes_at_landmarks"][f"{pct}%"][f"w{w}"]
                assert (x is None) == (y is None) and (x is None or abs(x - y) <= 1e-9 * max(abs(x), 1e-6)), (key, pct, w, x, y)
        ra, rb = a[key]["rolling_stats"], b[key]["rolling_stats"]
        assert len(ra) == len(rb) == 40
        for x, y in zip(ra, rb):
            assert x["step_center"] == y["step_center"] and x["n"] == y["n"]
            assert abs(x["mean"] - y["mean"]) < 1e-12 and abs(x["std"] - y["std"]) < 1e-12
        assert abs(a[key]["stability_score"] - b[key]["stability_score"]) < 1e-9
        ja, jb = a[key]["jumps"], b[key]["jumps"]
        assert [j["step"] for j in ja] == [j["step"] for j in jb]
        assert all(abs(x["delta"] - y["delta"]) < 1e-12 and abs(x["sigma"] - y["sigma"]) <= 0.011 for x, y in zip(ja, jb))
    steps = [j["step"] for j in b["train/loss"]["jumps"]]
    assert 7000 in steps and 7010 in steps and 15000 in steps


def test_run_comparison_and_factorial_effects_match_the_reference_engine(ref):
    """Deltas against the first run and the per-figure winners of ``compare_runs``, and main effects, interaction and
    the sign-based label of the 2 x 2 factorial for every logged metric, against ``src/eval/run_analysis.py``."""
    import numpy as np
    theirs = importlib.import_module("src.eval.run_analysis")
    from kotodama_b200.eval import run_analysis as ours
    rng = np.random.default_rng(5)

    def run(gain: float, rank_gain: float) -> dict:
        d = {}
        for s in range(0, 6001, 50):
            d[s] = {"train/loss": float(2.5 - gain + 3.0 * np.exp(-s / 1500.0) + rng.normal(0, 0.003)),
                    "train/perplexity": float(np.exp(2.5 - gain)), "perf/tokens_per_sec": float(40000 + 1000 * gain),
                    "train/tokens_consumed": float(s * 2 ** 21)}
            if s % 500 == 0:
                d[s].update({"geo/rankme_last": float(60 + rank_gain + 0.002 * s), "geo/twonn_id": float(20 + rank_gain),
                             "geo/ww_alpha_mean": float(3.0 - gain)})
        return d
    runs = {"P3": run(0.0, 0.0), "NCA": run(0.10, 4.0), "P3-AR": run(0.05, -2.0), "NCA-AR": run(0.21, 2.5)}
    a, b = theirs.compare_runs(runs), ours.compare_runs(runs)
    assert a["baseline"] == b["baseline"] == "P3"
    for name, row in a["deltas"].items():
        for key, d in row.items():
            if d is None:
                assert key not in b["deltas"][name]
            else:
                assert abs(b["deltas"][name][key]["delta"] - d) < 1e-12, (name, key)
    assert a["best"] == b["best_per_metric"] and b["best"] == "NCA-AR"
    fa = theirs.factorial_analysis(runs, {"NCA": ("P3", "NCA"), "AttnRes": ("P3", "P3-AR")}, step=6000)
    fb = ours.factorial_analysis({(0, 0): runs["P3"], (1, 0): runs["NCA"], (0, 1): runs["P3-AR"], (1, 1): runs["NCA-AR"]},
                                 step=6000, all_metrics=True)
    mine = {"train/loss": fb, **fb["other_metrics"]}
    assert set(fa["effects"]) == set(mine)
    for key, e in fa["effects"].items():
        m = mine[key]
        assert abs(e["NCA_main"] - m["main_effect_a"]) < 1e-9 and abs(e["AttnRes_main"] - m["main_effect_b"]) < 1e-9, key
        assert abs(e["interaction"] - m["interaction"]) < 1e-9 and e["classification"] == m["additivity"], key
    assert fb["additivity"] == "sub-additive" and fb["classification"] == "reinforcing"       # both together gain more than the sum


def test_geometric_health_and_summary_comparison_match_the_reference_engine(ref):
    """Layer discovery, landmark steps snapped to steps that have geometric records, the per-layer profile at every
    landmark, the depth gradient at the last one and the RankMe stability figure; and the endpoint summary against a
    reference summary with the figures that moved by more than the threshold - against ``src/eval/run_analysis.py``."""
    import numpy as np
    theirs = importlib.import_module("src.eval.run_analysis")
    from kotodama_b200.eval import run_analysis as ours
    rng = np.random.default_rng(9)
    data = {}
    for s in range(0, 12001, 100):
        data[s] = {"train/loss": float(3.0 + 2.0 * np.exp(-s / 3000.0)), "train/perplexity": float(np.exp(3.0)),
                   "perf/tokens_per_sec": 38000.0, "train/tokens_consumed": float(s) * 2 ** 21}
        if s % 700 == 0:                                   # geometric records on a grid that misses the landmark steps
            data[s]["geo/rankme_last"] = float(80 - 30 * np.exp(-s / 2000.0) + rng.normal(0, 0.5 + 2.0 * np.exp(-s / 1500.0)))
            for layer in (0, 7, 14, 21, 27):
                for proj in ("q_proj", "k_proj", "o_proj", "gate_proj", "down_proj"):
                    data[s][f"geo/layer_{layer}/stable_rank_{proj}"] = float(10 + layer + rng.normal(0, 0.1))
                data[s][f"geo/layer_{layer}/attn_entropy_mean"] = float(3.0 - 0.02 * layer + rng.normal(0, 0.01))
                data[s][f"geo/layer_{layer}/attn_entropy_std"] = float(0.3 + rng.normal(0, 0.01))
                data[s][f"geo/layer_{layer}/anisotropy"] = float(0.1 + 0.01 * layer)
                data[s][f"geo/layer_{layer}/dead_units"] = 0.0
    a, b = theirs.geometric_health(data), ours.geometric_health(data)
    assert a["layers"] == sorted(b["layers"]) == [0, 7, 14, 21, 27] and a["landmarks"] == b["landmarks"]
    for lm, prof in a["profiles"].items():
        assert prof["step"] == b["profiles"][lm]["step"]
        for layer in a["layers"]:
            assert prof[f"layer_{layer}"] == b["profiles"][lm][f"layer_{layer}"], (lm, layer)
    assert a["depth_gradient"] == b["depth_gradient"] and abs(a["rankme_stability"] - b["rankme_stability"]) < 1e-12
    other = {s: {**v, "train/loss": v["train/loss"] * 1.2} for s, v in data.items()}
    target = theirs.endpoint_summary(other)
    ca, cb = theirs.reference_comparison(data, target, threshold_pct=5.0), ours.reference_comparison(data, target, threshold_pct=5.0)
    assert ca == cb and {f["metric"] for f in cb["flagged"]} >= {"loss_final", "loss_min"}


def test_checkpoint_registry_loader_and_generation_match_the_reference_eval_modules(ref, tmp_path):
    """``src/eval/model_loader.py`` and ``src/eval/generate.py`` against this package's evaluation helpers: the
    reference's own grouped ``configs/checkpoints.yaml`` gives the same entries (paths, groups, tags, AttnRes settings),
    its ``configs/model.yaml`` the same shapes, one checkpoint (with wrapper prefixes, AttnRes with explicit
    boundaries) loads into the same weights and logits through both loaders - explicitly configured and auto-detected -
    and seeded sampling (temperature, nucleus, end-of-sequence set, length limit) draws the same tokens."""
    import yaml
    loader = importlib.import_module("src.eval.model_loader")
    gen = importlib.import_module("src.eval.generate")
    from kotodama_b200 import eval as ours
    refdir = os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
    reg_file = os.path.join(refdir, "configs", "checkpoints.yaml")
    if not os.path.isfile(reg_file):
        pytest.skip("the reference's configs are not on this machine")
    a, b = loader.load_checkpoint_registry(reg_file), ours.load_checkpoint_registry(reg_file)
    assert list(a) == list(b) and len(a) >= 5
    for name, e in a.items():
        assert str(e.path) == b[name].path and e.group == b[name].group and e.tags == b[name].tags
        assert e.attn_res_config == b[name].attn_res_config, name
    for section in ("proxy", "intermediate", "model"):
        theirs_kw = loader.load_model_config(os.path.join(refdir, "configs", "model.yaml"), section)
        mine = ours.load_model_config(os.path.join(refdir, "configs", "model.yaml"), section)
        assert all(getattr(mine, k) == v for k, v in theirs_kw.items() if hasattr(mine, k)), section
    # one small model under both loaders
    shape = dict(hidden_size=64, num_layers=6, num_attention_heads=4, num_kv_heads=2, head_dim=16, intermediate_size=128,
                 vocab_size=211, max_position_embeddings=128)
    model_yaml = tmp_path / "model.yaml"
    model_yaml.write_text(yaml.safe_dump({"proxy": {**shape, "attn_impl": "sdpa"}}))       # no flash-attention library on the CPU
    torch.manual_seed(0)
    src_model = ref.llama.LuxiaBaseModel(ref.llama.LuxiaModelConfig(**shape, attn_impl="sdpa", attn_res=True,
                                                                    attn_res_boundaries=[0, 2, 5]))
    with torch.no_grad():
        for n, p_ in src_model.named_parameters():
            if "res_query" in n:
                p_.normal_(0, 0.3)
    ck = tmp_path / "step_00000010.pt"
    torch.save({"step": 10, "model": {"_orig_mod.module." + k: v for k, v in src_model.state_dict().items()}}, ck)
    explicit = {"attn_res": True, "attn_res_boundaries": [0, 2, 5]}
    ids = torch.randint(0, 211, (1, 12), generator=torch.Generator().manual_seed(1))
    for cfg_kw in (explicit, None):
        m_a = loader.load_model(ck, config_path=model_yaml, config_section="proxy", attn_res_config=cfg_kw, device="cpu")
        m_b, meta = ours.load_model(ck, config_path=str(model_yaml), section="proxy", attn_res_config=cfg_kw, device="cpu")
        assert meta["step"] == 10 and m_b.config.attn_res and sorted(m_b.config.boundaries()) == sorted(m_a._attn_res_boundary_set)
        sd_a, sd_b = m_a.state_dict(), m_b.state_dict()
        assert list(sd_a) == list(sd_b) and all(torch.equal(sd_a[k], sd_b[k]) for k in sd_a)
        with torch.no_grad():
            assert torch.allclose(m_a(ids)["logits"], m_b(ids)["logits"], atol=1e-5)
    for kw in (dict(temperature=0.9, top_p=None), dict(temperature=0.7, top_p=0.8), dict(temperature=1.3, top_p=0.95)):
        torch.manual_seed(7)
        out_a = gen.generate(m_a, ids, max_new_tokens=24, eos_tokens=[3, 5], max_seq_len=30, **kw)
        torch.manual_seed(7)
        out_b = ours.generate(m_b, ids, max_new_tokens=24, top_k=0, eos_tokens=[3, 5], max_seq_len=30, **kw)
        assert out_a.tolist() == out_b.tolist() and (out_a.shape[1] == 30 or int(out_a[0, -1]) in (3, 5)), kw


def test_http_routes_answer_like_the_reference_server(ref):
    """The same requests to the reference's FastAPI app (its globals pointed at a small model) and to this package's
    app (paged engine) on the same weights: ``/health``, ``/v1/models``, ``/info``, ``/generate`` (plain, with a stop
    string, streamed), ``/v1/completions`` (n = 2, stop as a string) and the validation errors - same status codes,
    same keys, and with greedy decoding the same text, token counts, stream frames and usage figures."""
    import importlib.util
    import json
    fastapi_testclient = pytest.importorskip("fastapi.testclient")
    serve_py = os.path.join(os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference")), "serve.py")
    if not os.path.isfile(serve_py):
        pytest.skip("the reference's serve.py is not on this machine")
    spec = importlib.util.spec_from_file_location("reference_serve_app", serve_py)
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)
    from kotodama_b200.serve.app import create_app
    from kotodama_b200.serve.engine import ServingEngine
    m_a, m_b = _pair(ref, dtype=torch.float32, boundaries=[0, 1, 3])
    m_b.load_state_dict(m_a.state_dict())
    m_a.eval(), m_b.eval()

    class Letters:                                # id -> one letter, so every token is one character of text
        eos_token_id, bos_token_id, vocab_size, name = 210, 209, 211, "letters"

        def encode(self, text, return_tensors=None):
            ids = [ord(c) - 97 for c in text]
            return torch.tensor([ids]) if return_tensors == "pt" else ids

        def decode(self, ids, skip_special_tokens=True):
            return "".join(chr(97 + int(i) % 26) for i in ids)
    theirs._model, theirs._tokenizer, theirs._device = m_a, Letters(), torch.device("cpu")
    ca = fastapi_testclient.TestClient(theirs.app)                      # no context manager: its start-up hook would load a checkpoint
    eng = ServingEngine(m_b, device="cpu", dtype=torch.float32, max_batch=4, max_ctx=m_b.config.max_position_embeddings)
    app = create_app(eng, Letters(), model_name="luxia-base-proxy-ddv1")
    with fastapi_testclient.TestClient(app) as cb:
        ha, hb = ca.get("/health").json(), cb.get("/health").json()
        assert ha["status"] == hb["status"] == "ok"
        ma, mb = ca.get("/v1/models").json(), cb.get("/v1/models").json()
        assert ma["object"] == mb["object"] and set(ma["data"][0]) <= set(mb["data"][0]) and ma["data"][0]["id"] == mb["data"][0]["id"]
        ia, ib = ca.get("/info").json(), cb.get("/info").json()
        assert set(ia) <= set(ib) and ia["params"] == ib["params"] and ia["name"] == ib["name"]
        assert set(ia["config"]) <= set(ib["config"]) and all(ib["config"][k] == v for k, v in ia["config"].items() if k != "attn_impl")
        body = {"prompt": "thequickbrownfox", "max_new_tokens": 12, "temperature": 0.0}
        ga, gb = ca.post("/generate", json=body), cb.post("/generate", json=body)
        assert ga.status_code == gb.status_code == 200 and set(ga.json()) == set(gb.json())
        for k in ("text", "prompt_tokens", "completion_tokens"):
            assert ga.json()[k] == gb.json()[k], k
        text = ga.json()["text"]
        stop = {**body, "stop_strings": [text[4:6]], "repetition_penalty": 1.0}
        sa, sb = ca.post("/generate", json=stop).json(), cb.post("/generate", json=stop).json()
        assert sa["text"] == sb["text"] and sa["completion_tokens"] == sb["completion_tokens"] < 12
        pen = {**body, "repetition_penalty": 1.7}
        assert ca.post("/generate", json=pen).json()["text"] == cb.post("/generate", json=pen).json()["text"]

        def frames(client):
            with client.stream("POST", "/generate", json={**body, "stream": True}) as r:
                return [json.loads(l[6:]) for l in r.iter_lines() if l.startswith("data: ")]
        fa, fb = frames(ca), frames(cb)
        assert "".join(f["token"] for f in fa[:-1]) == "".join(f["token"] for f in fb[:-1]) == text
        assert fa[-1] == {k: fb[-1][k] for k in fa[-1]} and fa[-1]["done"] is True
        oai = {"prompt": "lazydog", "max_tokens": 9, "n": 2, "temperature": 0.0, "frequency_penalty": 0.4, "stop": text[1:2]}
        oa, ob = ca.post("/v1/completions", json=oai), cb.post("/v1/completions", json=oai)
        assert oa.status_code == ob.status_code == 200
        oa, ob = oa.json(), ob.json()
        assert set(oa) <= set(ob) and oa["object"] == ob["object"] and oa["model"] == ob["model"] and oa["usage"] == ob["usage"]
        assert [(c["text"], c["index"], c["finish_reason"]) for c in oa["choices"]] == [(c["text"], c["index"], c["finish_reason"]) for c in ob["choices"]]
        for bad in ({"prompt": "a", "temperature": 3.0}, {"prompt": "a", "max_new_tokens": 0}, {"prompt": "a", "repetition_penalty": 0.5},
                    {"max_new_tokens": 4}):
            assert ca.post("/generate", json=bad).status_code == cb.post("/generate", json=bad).status_code == 422, bad
        long = {"prompt": "a" * (m_b.config.max_position_embeddings + 3)}
        assert ca.post("/generate", json=long).status_code == cb.post("/generate", json=long).status_code == 400
    app.state.worker.shutdown()


def test_nca_generator_command_line_takes_the_reference_flags(ref, tmp_path):
    """Every flag of the reference's ``python -m src.nca.generator`` exists here with the same default, and a small
    generation + ``--verify <path>`` runs through this package's command line."""
    import re
    from kotodama_b200.nca import generator as ours
    src = open(os.path.join(REF, "nca", "generator.py")).read()
    theirs = {m.group(1): m.group(2) for m in re.finditer(r'add_argument\(\s*"--(\w+)"([^)]*)\)', src)}
    assert len(theirs) >= 20
    own = open(ours.__file__).read()
    mine = {m.group(1): m.group(2) for m in re.finditer(r'add_argument\(\s*"--(\w+)"([^)]*)\)', own)}
    for flag, rest in theirs.items():
        assert flag in mine, flag
        d = re.search(r"default=([^,\s)]+)", rest)
        if d and flag not in ("device", "verify", "output"):
            assert re.search(r"default=([^,\s)]+)", mine[flag]).group(1) == d.group(1), flag
    out = tmp_path / "nca.bin"
    ours.main(["--output", str(out), "--tokens", "3000", "--num_rules", "2", "--sims_per_rule", "1", "--grid_size", "8", "--d_state", "3",
               "--n_groups", "1", "--num_steps", "6", "--burn_in", "2", "--kernel_size", "5", "--hidden_dim", "8", "--num_hidden_layers", "1",
               "--identity_bias", "0.5", "--temperature", "0.8", "--gzip_lower", "0.0", "--gzip_upper", "1.0", "--no_mixed", "--device", "cpu",
               "--seed", "1", "--verify"])
    rep = ours.verify_file(out, ours.NCAConfig(grid_size=8, d_state=3, n_groups=1))
    assert 0 < rep["tokens"] <= 3000 and rep["in_vocab"] and rep["max_id"] < 3 ** 4 + 2
    ours.main(["--verify", str(out), "--d_state", "3", "--grid_size", "8", "--n_groups", "1"])


def test_command_line_tools_take_the_reference_scripts_flags():
    """Every ``--flag`` of the reference's utility, analysis and serving scripts is accepted by its counterpart here
    (read from the parsers' source; shared checkpoint arguments live in ``tools/analysis/_common.py``)."""
    import re
    refdir = os.environ.get("KOTODAMA_REFERENCE", os.path.join(os.path.dirname(ROOT), "reference"))
    if not os.path.isdir(os.path.join(refdir, "scripts", "analysis")):
        pytest.skip("the reference's scripts are not on this machine")
    pairs = {"scripts/utils/" + f: "tools/" + f for f in ("tokenize_data.py", "smoke_test.py", "profile_step.py", "pull_metrics.py",
                                                          "visualize_nca.py")}
    pairs["serve.py"] = "serve.py"
    pairs.update({"scripts/analysis/" + f: "tools/analysis/" + f for f in os.listdir(os.path.join(refdir, "scripts", "analysis"))
                  if f.endswith(".py")})
    common = open(os.path.join(ROOT, "tools", "analysis", "_common.py")).read()
    checked = 0
    for theirs, mine in pairs.items():
        flags = set(re.findall(r'add_argument\(\s*(?:"-\w",\s*)?"(--[\w-]+)"', open(os.path.join(refdir, theirs)).read()))
        own = open(os.path.join(ROOT, mine)).read() + (common if "analysis" in mine else "")
        missing = sorted(f for f in flags if f'"{f}"' not in own)
        assert not missing, (mine, missing)
        checked += len(flags)
    assert checked >= 100
