"""Evaluation helpers: loader, state-exposing forward, generation, perplexity, metrics analysis."""
import json

import numpy as np
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.eval import (compute_perplexity, extract_series, forward_with_states, generate, get_nearest_step,
                                load_metrics, load_model, run_analysis)
from kotodama_b200.models.llama import KotodamaModel


def _model(attn_res=True):
    torch.manual_seed(0)
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=attn_res, attn_res_n_blocks=2)
    m = KotodamaModel(cfg).eval()
    with torch.no_grad():
        for n, p in m.named_parameters():
            if "query" in n:
                p.normal_(0, 0.3)
    return cfg, m


def test_forward_with_states_matches_model_and_exposes_routes():
    for attn_res in (True, False):
        cfg, m = _model(attn_res)
        ids = torch.randint(0, cfg.vocab_size, (2, 24))
        res = forward_with_states(m, ids, attention_layers=[1])
        assert torch.allclose(res.logits, m(ids)["logits"], atol=1e-5)
        assert len(res.states) == cfg.num_layers + 1 and res.attention[1].shape == (2, 4, 24, 24)
        assert torch.allclose(res.attention[1].sum(-1), torch.ones(2, 4, 24), atol=1e-5)
        if attn_res:
            assert abs(float(res.route_weights["final"].sum()) - 1) < 1e-5 and "mlp_3" in res.route_weights


def test_load_model_autodetects_attnres_and_generate(tmp_path):
    cfg, m = _model()
    torch.save({"model": {("_orig_mod." + k): v for k, v in m.state_dict().items()}, "step": 7}, tmp_path / "c.pt")
    loaded, meta = load_model(tmp_path / "c.pt", section="smoke", attn_res_boundaries=None)
    loaded.config.attn_res_n_blocks = 2
    assert loaded.config.attn_res and meta["step"] == 7
    cfg2 = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    loaded, _ = load_model(tmp_path / "c.pt", config=cfg2)
    ids = torch.randint(0, cfg.vocab_size, (1, 8))
    a = generate(loaded, ids, max_new_tokens=6, temperature=0.0)
    b = generate(m, ids, max_new_tokens=6, temperature=0.0, use_cache=False)
    assert a.shape == (1, 14) and torch.equal(a, b)


def test_perplexity_and_metrics_analysis(tmp_path):
    cfg, m = _model()
    toks = np.random.default_rng(0).integers(0, cfg.vocab_size, 4000).astype("<u2")
    toks.tofile(tmp_path / "d.bin")
    r = compute_perplexity(m, tmp_path / "d.bin", seq_len=64, max_tokens=2048, batch_size=4)
    assert r["tokens"] == 32 * 63 and 100 < r["perplexity"] < 5000
    with open(tmp_path / "m.jsonl", "w") as fh:
        for s in range(0, 2000, 10):
            fh.write(json.dumps({"step": s, "timestamp": 0, "train/loss": 5.0 - 0.001 * s,
                                 "train/perplexity": 100.0, "perf/tokens_per_sec": 1000.0}) + "\n")
            if s % 500 == 0:
                fh.write(json.dumps({"step": s, "geo/rankme_last": 50 + s / 100,
                                     "geo/layer_0/stable_rank_q_proj": 10.0, "geo/layer_0/dead_units": 0.0}) + "\n")
        fh.write("not json\n")
    data = load_metrics(tmp_path / "m.jsonl")
    assert len(data) == 200 and "geo/rankme_last" in data[500] and "train/loss" in data[500]
    assert get_nearest_step(data, 503) == 500 and get_nearest_step({1: {}}, 5000) is None
    assert extract_series(data, "geo/rankme_last")[0] == (0, 50.0)
    summ = run_analysis.endpoint_summary(data)
    assert summ["max_step"] == 1990 and abs(summ["loss_final"] - 3.01) < 1e-9 and summ["rankme_final"] == 65.0
    dyn = run_analysis.training_dynamics(data)
    assert abs(dyn["train/loss"]["slopes"]["last_500"] + 0.001) < 1e-9 and dyn["train/loss"]["jumps"] == []
    lm = dyn["train/loss"]["slopes_at_landmarks"]["50%"]
    assert abs(lm["w100"] + 0.001) < 1e-9 and abs(lm["w500"] + 0.001) < 1e-9          # a straight line: same slope at every scale
    assert dyn["train/loss"]["inflection_points"] == [] and dyn["train/loss"]["rolling_stats"][0]["p25"] < dyn["train/loss"]["rolling_stats"][0]["p75"]
    assert 0.5 < dyn["train/loss"]["stability_score"] < 2.0
    gh = run_analysis.geometric_health(data)
    assert 0 in gh["layers"] and gh["flags"] == []
    assert gh["landmarks"]["final"] == 1500 and gh["profiles"]["mid"]["layer_0"]["stable_rank_q_proj"] == 10.0
    worse = {s: {"train/loss": v["train/loss"] + 0.5} for s, v in data.items() if "train/loss" in v}
    cmp_ = run_analysis.compare_runs({"a": data, "b": worse})
    assert cmp_["best"] == "a" and cmp_["baseline"] == "a"
    assert cmp_["deltas"]["b"]["loss_final"]["verdict"] == "worse" and abs(cmp_["deltas"]["b"]["loss_final"]["delta"] - 0.5) < 1e-9
    fa = run_analysis.factorial_analysis({(0, 0): worse, (0, 1): data, (1, 0): data, (1, 1): data})
    assert abs(fa["interaction"] - 0.5) < 1e-9
    # either factor alone gains 0.5, both together gain 0.5 too: the second factor adds nothing on top of the first
    assert fa["classification"] == "offsetting" and abs(fa["additive_prediction"] - (fa["values"]["00"] - 1.0)) < 1e-9
    better2 = {s: {"train/loss": v["train/loss"] - 0.5} for s, v in data.items() if "train/loss" in v}
    assert run_analysis.factorial_analysis({(0, 0): worse, (0, 1): data, (1, 0): data, (1, 1): better2})["classification"] == "additive"
    rc = run_analysis.reference_comparison(data, worse)
    assert rc["metrics"]["train/loss"]["delta"] < 0 and rc["steps_to_reference_final_loss"] < 1990
    assert abs(rc["landmarks"]["50%"]["delta"]["train/loss"] + 0.5) < 1e-9
    # a curve that bends: fast early, flat late -> one inflection-free decay but a plateau and a stability score below 1
    bend = {s: {"train/loss": 2.0 + 3.0 * 0.995 ** s + (0.05 if s < 500 and s % 20 == 0 else 0.0)} for s in range(0, 4000, 10)}
    d2 = run_analysis.training_dynamics(bend, ["train/loss"])["train/loss"]
    assert d2["stability_score"] < 0.5 and d2["plateaus"] and abs(d2["slopes"]["last_1000"]) < 1e-4
