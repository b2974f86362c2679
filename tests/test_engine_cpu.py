"""The hand-scheduled executor must produce the gradients autograd produces for the plain
model, and its optimizer step must match the stand-alone Muon/AdamW optimizers."""
import copy

import pytest
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.engine import TrainEngine
from kotodama_b200.models.llama import KotodamaModel
from kotodama_b200.optim.muon import build_hybrid_optimizer


def small_cfg(attn_res=True, **kw):
    base = dict(hidden_size=64, num_layers=4, num_attention_heads=4, num_kv_heads=2, head_dim=16,
                intermediate_size=96, vocab_size=97, max_position_embeddings=64, attn_res=attn_res,
                attn_res_n_blocks=2, z_loss_weight=1e-3)
    base.update(kw)
    return ModelConfig(**base)


def randomise(model, seed=0):
    g = torch.Generator().manual_seed(seed)
    with torch.no_grad():
        for n, p in model.named_parameters():
            if "query" in n:
                p.copy_(torch.randn(p.shape, generator=g) * 0.3)
            elif p.ndim == 1:
                p.copy_(1 + 0.1 * torch.randn(p.shape, generator=g))
            else:
                p.copy_(torch.randn(p.shape, generator=g) * 0.08)


@pytest.mark.parametrize("attn_res,boundaries", [(True, None), (True, [0, 1, 3]), (True, [1, 2]), (False, None)])
def test_engine_grads_match_autograd(attn_res, boundaries):
    torch.manual_seed(0)
    cfg = small_cfg(attn_res, attn_res_boundaries=boundaries)
    ref = KotodamaModel(cfg).double()
    randomise(ref)
    model = copy.deepcopy(ref)
    ids = torch.randint(0, cfg.vocab_size, (3, 24))
    out = ref(ids, labels=ids)
    out["loss"].backward()
    eng = TrainEngine(model, device="cpu", dtype=torch.float64)
    loss, zl = eng.forward_backward(ids)
    assert torch.allclose(loss, out["loss"], rtol=1e-9, atol=1e-10)
    assert torch.allclose(zl, out["z_loss"], rtol=1e-9, atol=1e-12)
    for (n, p), (_, q) in zip(ref.named_parameters(), model.named_parameters()):
        g = p.grad if p.grad is not None else torch.zeros_like(p)
        assert torch.allclose(q.grad, g, rtol=1e-7, atol=1e-9), n


@pytest.mark.parametrize("layers,boundaries", [(8, None), (28, [0, 3, 7, 12, 21, 25]), (6, [2, 4])])
def test_blocked_routing_matches_stacked(layers, boundaries):
    """The blocked AttnRes schedule (one phase-1 pass per block for all of its queries, a phase-2
    merge per sub-layer) equals the stacked per-call form and autograd, fp64, uniform and explicit
    boundaries."""
    torch.manual_seed(1)
    cfg = small_cfg(True, num_layers=layers, attn_res_n_blocks=4, attn_res_boundaries=boundaries, hidden_size=32,
                    intermediate_size=48, num_attention_heads=2, num_kv_heads=1)
    ref = KotodamaModel(cfg).double()
    randomise(ref)
    m_blocked, m_plain = copy.deepcopy(ref), copy.deepcopy(ref)
    ids = torch.randint(0, cfg.vocab_size, (2, 12))
    out = ref(ids, labels=ids)
    out["loss"].backward()
    eng = TrainEngine(m_blocked, device="cpu", dtype=torch.float64)
    assert eng._route_groups and all(g["S"] >= 2 for g in eng._route_groups)
    n_blocked = sum(len(g["members"]) for g in eng._route_groups)
    assert n_blocked == len(eng._route_plan) >= 5
    plain = TrainEngine(m_plain, device="cpu", dtype=torch.float64)
    plain._route_plan, plain._route_groups = {}, []
    l1, _ = eng.forward_backward(ids)
    l2, _ = plain.forward_backward(ids)
    assert torch.allclose(l1, out["loss"], rtol=1e-10) and torch.allclose(l2, out["loss"], rtol=1e-10)
    assert torch.allclose(eng.arena.grads, plain.arena.grads, rtol=1e-7, atol=1e-10)
    for (n, p), (_, q) in zip(ref.named_parameters(), m_blocked.named_parameters()):
        g = p.grad if p.grad is not None else torch.zeros_like(p)
        assert torch.allclose(q.grad, g, rtol=1e-7, atol=1e-9), n


def test_engine_grad_accumulation_matches_big_batch():
    cfg = small_cfg()
    m1 = KotodamaModel(cfg).double(); randomise(m1)
    m2 = copy.deepcopy(m1)
    ids = torch.randint(0, cfg.vocab_size, (4, 16))
    e1 = TrainEngine(m1, device="cpu", dtype=torch.float64)
    e2 = TrainEngine(m2, device="cpu", dtype=torch.float64)
    e1.forward_backward(ids, 1.0)
    e2.forward_backward(ids[:2], 0.5, first_micro=True, last_micro=False)
    e2.forward_backward(ids[2:], 0.5, first_micro=False, last_micro=True)
    assert torch.allclose(e1.arena.grads, e2.arena.grads, rtol=1e-8, atol=1e-10)


def test_engine_step_matches_reference_optimizers():
    cfg = small_cfg()
    ref = KotodamaModel(cfg); randomise(ref)
    model = copy.deepcopy(ref)
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    muon, adamw = build_hybrid_optimizer(ref, muon_lr=0.02, adamw_lr=1e-3)
    eng = TrainEngine(model, device="cpu", dtype=torch.float32, muon_lr=0.02, adamw_lr=1e-3, gradient_clip=1.0)
    for _ in range(3):
        out = ref(ids, labels=ids)
        out["loss"].backward()
        torch.nn.utils.clip_grad_norm_(ref.parameters(), 1.0)
        muon.step(); adamw.step()
        muon.zero_grad(); adamw.zero_grad()
        res = eng.train_step([ids])
        assert abs(float(res["loss"]) - float(out["loss"].detach())) < 2e-4
    for (n, p), (_, q) in zip(ref.named_parameters(), model.named_parameters()):
        assert torch.allclose(p, q, rtol=2e-3, atol=1e-3), n  # fp16 Newton-Schulz amplifies rounding-order differences


def test_arena_keeps_reference_parameter_order_and_fused_views():
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    model = KotodamaModel(cfg)
    names = [n for n, _ in model.named_parameters()]
    assert names[:2] == ["final_res_query", "embed_tokens.weight"]
    assert names[2:6] == ["layers.0.attn_res_query", "layers.0.mlp_res_query", "layers.0.attn_norm.weight",
                          "layers.0.attn.q_proj.weight"]
    assert names[-2:] == ["norm.weight", "final_res_norm.weight"]
    eng = TrainEngine(model, device="cpu")
    assert [n for n, _ in model.named_parameters()] == names
    w = eng.layer_w[1]["wqkv"]
    assert w.shape == ((4 + 2 * 2) * 64, 256)
    assert w.data_ptr() == model.layers[1].attn.q_proj.weight.data_ptr()
    assert torch.equal(w[4 * 64: 6 * 64], model.layers[1].attn.k_proj.weight)
    assert torch.equal(eng.layer_w[1]["wgu"][512:], model.layers[1].ffn.up_proj.weight)
    sd = model.state_dict()
    assert "layers.0.attn.q_proj.weight" in sd and "rope_cos" not in sd


def test_fp8_block_scaled_training_tracks_full_precision():
    """--fp8: projections run through the block-scaled e4m3 path (quantisers + scaled GEMM, here the
    PyTorch restatement); losses stay close to the unquantised run and fall."""
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    batch = torch.randint(0, cfg.vocab_size, (2, 128), generator=torch.Generator().manual_seed(1))

    def run(fp8):
        torch.manual_seed(0)
        eng = TrainEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32, muon_lr=0.02, adamw_lr=1e-3, fp8=fp8)
        if fp8:
            from kotodama_b200.ops.reference import Fp8Weight
            assert isinstance(eng.layer_w[0]["wqkv"], Fp8Weight) and eng.layer_w[0]["wqkv"].q.dtype == torch.float8_e4m3fn
        return [float(eng.train_step([batch])["loss"]) for _ in range(4)]

    full, q = run(False), run(True)
    assert q[-1] < q[0] - 2.0
    for a, b in zip(full, q):
        assert abs(a - b) < 0.05, (full, q)
    assert full != q
