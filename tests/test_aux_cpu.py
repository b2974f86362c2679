"""NCA generator, geometric monitor, datasets, checkpoints, scheduler, logger."""
import json
import os

import numpy as np
import pytest
import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.models.llama import KotodamaModel


# ------------------------------------------------------------------ NCA
def test_nca_tokenisation_and_simulation():
    from kotodama_b200.nca.generator import (NCAConfig, NCARule, compute_gzip_complexity, generate_nca_dataset,
                                             simulate_trajectory, tokenize_trajectory)
    cfg = NCAConfig(grid_size=8, d_state=3, n_groups=2, num_steps=4, burn_in=2, filter_enabled=False,
                    mixed_complexity=False, hidden_dim=8)
    assert cfg.vocab_size == 3 ** 4 + 2 and cfg.tokens_per_frame == 16 + 2 and cfg.tokens_per_timestep == 36
    torch.manual_seed(0)
    rule = NCARule(3, 2, 3, 8, 2)
    traj = simulate_trajectory(rule, 8, 3, 2, 4, 2, 1.0, 0.5, batch_size=2)
    assert traj.shape == (2, 4, 2, 8, 8) and int(traj.max()) < 3 and int(traj.min()) >= 0
    toks = tokenize_trajectory(traj, 3, 2)
    assert toks.dtype == np.uint16 and len(toks) == 2 * cfg.tokens_per_trajectory
    # hand-check the first frame: START, 16 patch codes, END
    assert toks[0] == 81 and toks[17] == 82
    g = traj[0, 0, 0]
    code = int(g[0, 0]) + 3 * int(g[0, 1]) + 9 * int(g[1, 0]) + 27 * int(g[1, 1])
    assert toks[1] == code
    code_next = int(g[0, 2]) + 3 * int(g[0, 3]) + 9 * int(g[1, 2]) + 27 * int(g[1, 3])
    assert toks[2] == code_next
    assert 0 < compute_gzip_complexity(toks) < 1.5


def test_nca_dataset_file(tmp_path):
    from kotodama_b200.data.dataset import TokenizedDataset, verify_token_file
    from kotodama_b200.nca.generator import NCAConfig, generate_nca_dataset
    cfg = NCAConfig(grid_size=8, d_state=3, n_groups=2, num_steps=4, burn_in=1, filter_enabled=False, hidden_dim=8)
    out = tmp_path / "nca.bin"
    n = generate_nca_dataset(cfg, out, max_tokens=500, num_rules=3, sims_per_rule=2)
    assert n == 500 and out.stat().st_size == 1000
    info = verify_token_file(str(out), cfg.vocab_size)
    assert info["tokens"] == 500 and info["in_vocab"]
    ds = TokenizedDataset(str(out), seq_len=50, rank=0, world_size=2, seed=1)
    first = next(iter(ds))
    assert first.dtype == torch.long and first.shape == (50,)


# ------------------------------------------------------------------ datasets
def test_random_dataset_resumable_and_rank_distinct():
    from kotodama_b200.data.dataset import BatchIterator, RandomTokenDataset
    a = RandomTokenDataset(1000, 16, seed=3, rank=0)
    it = iter(a)
    x0, x1 = next(it), next(it)
    state = a.state_dict()
    x2 = next(it)
    b = RandomTokenDataset(1000, 16, seed=3, rank=0)
    b.load_state_dict(state)
    assert torch.equal(next(iter(b)), x2) and not torch.equal(x0, x1)
    c = RandomTokenDataset(1000, 16, seed=3, rank=1)
    assert not torch.equal(next(iter(c)), x0)
    batch = next(BatchIterator(RandomTokenDataset(1000, 16, fixed=True), 4))
    assert batch.shape == (4, 16) and int(batch.max()) < 1000


def test_tokenized_dataset_partitions_ranks(tmp_path):
    from kotodama_b200.data.dataset import TokenizedDataset, write_token_file
    path = tmp_path / "t.bin"
    write_token_file(str(path), np.arange(1000) % 60000)
    seen = []
    for r in range(2):
        ds = TokenizedDataset(str(path), seq_len=100, rank=r, world_size=2, seed=5)
        it = iter(ds)
        seen.append({int(next(it)[0]) for _ in range(5)})
    assert seen[0].isdisjoint(seen[1]) and len(seen[0] | seen[1]) == 10
    with pytest.raises(ValueError):
        write_token_file(str(path), [70000])


# ------------------------------------------------------------------ schedule
def test_wsd_schedule_and_presets():
    from kotodama_b200.optim.muon import NS_COEFFICIENT_PRESETS, HybridScheduler, NoOpOptimizer, resolve_ns_coefficients

    class Opt:
        def __init__(self, lr):
            self.defaults = {"lr": lr}; self.param_groups = [{"lr": lr}]
    m, a = Opt(0.03), Opt(6e-4)
    s = HybridScheduler(m, a, warmup_steps=10, total_steps=100, decay_start_pct=0.9, decay_type="sqrt")
    assert s.get_lr_multiplier(0) == 0 and s.get_lr_multiplier(5) == 0.5 and s.get_lr_multiplier(50) == 1.0
    assert abs(s.get_lr_multiplier(95) - (1 - 0.5 ** 0.5)) < 1e-9 and s.decay_start_step == 90
    s.step(5)
    assert abs(m.param_groups[0]["lr"] - 0.015) < 1e-12 and abs(s.get_last_lr()["adamw_lr"] - 3e-4) < 1e-12
    assert HybridScheduler(m, a, 10, 100, 0.9, "linear").get_lr_multiplier(95) == 0.5
    assert abs(HybridScheduler(m, a, 10, 100, 0.9, "cosine").get_lr_multiplier(95) - 0.5) < 1e-3
    assert len(resolve_ns_coefficients("gram_ns", 7)) == 7 and resolve_ns_coefficients(None, 5)[0] == (3.4445, -4.7750, 2.0315)
    assert abs(NS_COEFFICIENT_PRESETS["polar_express"][0][0] - 8.28721201814563 / 1.05) < 1e-12
    with pytest.raises(ValueError):
        resolve_ns_coefficients("nope", 5)
    assert NoOpOptimizer().state_dict() == {}


def test_newton_schulz_orthogonalises():
    from kotodama_b200.optim.muon import newton_schulz_orthogonalize
    torch.manual_seed(0)
    for shape in ((32, 64), (64, 32), (3, 16, 48)):
        o = newton_schulz_orthogonalize(torch.randn(shape), 5, "original").float()
        s = torch.linalg.svdvals(o)
        assert float(s.min()) > 0.3 and float(s.max()) < 1.3, (shape, s.min(), s.max())


# ------------------------------------------------------------------ checkpoints
def _engine(tmp=None):
    from kotodama_b200.engine import TrainEngine
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    return cfg, model, TrainEngine(model, device="cpu", dtype=torch.float32)


def test_checkpoint_format_roundtrip_and_reference_optimizer_compat(tmp_path):
    from kotodama_b200.ckpt.manager import CheckpointManager
    from kotodama_b200.optim.muon import HybridScheduler, build_hybrid_optimizer
    cfg, model, eng = _engine()
    ids = torch.randint(0, cfg.vocab_size, (2, 32))
    eng.train_step([ids]); eng.train_step([ids])
    sched = HybridScheduler(eng.muon_opt, eng.adamw_opt, 2, 10)
    mgr = CheckpointManager(tmp_path, keep_last_n=2)
    for step in (1, 2, 3):
        mgr.save(step, model, eng.muon_opt, eng.adamw_opt, sched, tokens_consumed=step * 64, data_state={"position": step})
    assert sorted(p.name for p in tmp_path.glob("step_*.pt")) == ["step_00000002.pt", "step_00000003.pt"]
    assert not list(tmp_path.glob("*.tmp"))
    ck = torch.load(tmp_path / "step_00000003.pt", weights_only=False)
    assert set(ck["scheduler"]) == {"muon_base_lr", "adamw_base_lr", "warmup_steps", "total_steps", "decay_start_step",
                                   "decay_type"}
    assert len(ck["muon_optimizer"]["state"]) == 28 and len(ck["adamw_optimizer"]["state"]) == 36
    # the stand-alone (reference-layout) optimizers accept the saved state
    fresh = KotodamaModel(cfg)
    fresh.load_state_dict(ck["model"], strict=True)
    mu, ad = build_hybrid_optimizer(fresh)
    mu.load_state_dict(ck["muon_optimizer"]); ad.load_state_dict(ck["adamw_optimizer"])
    assert torch.allclose(mu.state[mu.param_groups[0]["params"][0]]["momentum_buffer"],
                          ck["muon_optimizer"]["state"][0]["momentum_buffer"])
    # and a fresh executor resumes bit-exactly
    cfg2, model2, eng2 = _engine()
    state = CheckpointManager(tmp_path).load_latest(model2, eng2.muon_opt, eng2.adamw_opt)
    assert state["step"] == 3 and state["data"] == {"position": 3}
    assert torch.equal(eng2.arena.params, eng.arena.params) and eng2.opt_step == eng.opt_step
    a, b = eng.train_step([ids]), eng2.train_step([ids])
    assert torch.equal(eng.arena.params, eng2.arena.params) and float(a["loss"]) == float(b["loss"])


def test_corrupt_checkpoint_is_skipped_and_async_manager_survives_write_error(tmp_path):
    from kotodama_b200.ckpt.manager import AsyncCheckpointManager, CheckpointManager
    from kotodama_b200.optim.muon import HybridScheduler
    cfg, model, eng = _engine()
    sched = HybridScheduler(eng.muon_opt, eng.adamw_opt, 2, 10)
    mgr = AsyncCheckpointManager(tmp_path / "ck", shm_dir=tmp_path / "shm", keep_last_n=3, compress=True)
    mgr.save(1, model, eng.muon_opt, eng.adamw_opt, sched)
    mgr.wait()
    assert (tmp_path / "ck" / "step_00000001.pt").exists() or (tmp_path / "ck" / "step_00000001.pt.zst").exists()
    # injected failure: the writer raises once; training-side calls do not
    real = mgr._write_shm
    calls = {"n": 0}

    def flaky(state, path):
        calls["n"] += 1
        if calls["n"] == 1:
            raise OSError("disk full (injected)")
        return real(state, path)
    mgr._write_shm = flaky
    mgr.save(2, model, eng.muon_opt, eng.adamw_opt, sched)
    mgr.save(3, model, eng.muon_opt, eng.adamw_opt, sched)
    mgr.shutdown()
    assert any("disk full" in e for e in mgr.errors)
    names = {p.name.split(".")[0] for p in (tmp_path / "ck").glob("step_*")}
    assert "step_00000003" in names and "step_00000002" not in names
    # truncated newest file: load falls back to the previous one
    newest = sorted((tmp_path / "ck").glob("step_00000003*"))[0]
    newest.write_bytes(newest.read_bytes()[:100])
    st = CheckpointManager(tmp_path / "ck").load_latest(model, eng.muon_opt, eng.adamw_opt)
    assert st is not None and st["step"] == 1


# ------------------------------------------------------------------ logger / monitor
def test_logger_jsonl_and_slopes(tmp_path):
    from kotodama_b200.monitor.logger import WandbLogger, format_step_line, linear_slope
    wb = WandbLogger(log_dir=str(tmp_path), use_wandb=False)
    for s in range(12):
        wb.log_step(s, loss=5.0 - 0.1 * s, z_loss=0.001, grad_norm=1.0, muon_lr=0.02, adamw_lr=1e-3,
                    tokens_per_sec=1000.0, tokens_consumed=s * 100, gpu_mem_gb=1.0, step_time_s=0.1)
    wb.log_geo(3, {"geo/rankme_last": 10.0})
    wb.finish()
    rows = [json.loads(l) for l in open(tmp_path / "metrics.jsonl")]
    assert {"train/loss", "train/perplexity", "optim/muon_lr", "perf/tokens_per_sec", "data/tokens_consumed_B"} <= set(rows[0])
    assert abs(rows[11]["train/loss_slope"] + 0.1) < 1e-6
    assert json.loads(open(tmp_path / "geo_metrics.jsonl").readline())["geo/rankme_last"] == 10.0
    assert linear_slope([(0, 1.0)]) == 0.0
    line = format_step_line(3, 10, 2.5, 0.001, 1.234, 0.02, 1e-3, 1234.0, 1.5, 2_000_000_000, 12.3)
    assert "tok/s=1234" in line and "gpu_mem=12.3GB" in line and "loss=2.5000" in line and "tokens=2.000B" in line


def test_geometric_monitor_tiers():
    from kotodama_b200.monitor.geometric import GeometricMonitor, MonitorConfig, rankme, stable_rank, twonn_id
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    mon = GeometricMonitor(model, MonitorConfig(tier2_twonn_samples=200))
    mon.set_probe_batch(torch.randint(0, cfg.vocab_size, (4, 32)))
    t1 = mon.tier1(0)
    assert t1["geo/rankme_last"] > 1 and "geo/layer_0/stable_rank_q_proj" in t1 and "geo/layer_3/attn_entropy_mean" in t1
    assert abs(sum(v for k, v in t1.items() if k.startswith("attnres/final_alpha/")) - 1.0) < 1e-4
    t2 = mon.tier2(0)
    assert "geo/ww_alpha_mean" in t2 and any(k.startswith("geo/twonn_id/") for k in t2)
    assert abs(rankme(torch.eye(8)) - 8) < 1e-3 and abs(stable_rank(torch.eye(8)) - 8) < 1e-3
    assert 1.0 < twonn_id(torch.randn(500, 3)) < 6.0
    # the probe forward is the model: its last entry (the final aggregation) under the output norm equals the model's
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    hidden, _ = mon._probe_forward(ids, set())
    ref, _ = model.hidden_states(ids)
    assert torch.allclose(model.norm(hidden[cfg.num_layers - 1]), ref, atol=1e-5)


def test_watchdog_names_rank_and_phase():
    import time
    from kotodama_b200.monitor.watchdog import StepWatchdog
    seen = []
    wd = StepWatchdog(0.15, rank=3, on_stall=lambda r, s, p, dt: seen.append((r, s, p)), poll_s=0.02)
    wd.phase(7, "data")
    time.sleep(0.05)
    wd.phase(7, "train_step")
    time.sleep(0.4)                                   # stalls in train_step
    wd.phase(8, "data")                               # heartbeat: the report is not repeated for the new phase
    time.sleep(0.05)
    wd.stop()
    assert seen == [(3, 7, "train_step")]
    assert wd.stalls[0][:2] == (7, "train_step") and wd.stalls[0][2] > 0.15
    off = StepWatchdog(0.0)
    off.phase(0, "x")
    off.stop()
    assert off._thread is None


def test_halt_on_nonfinite_stops_the_run(tmp_path, monkeypatch):
    from kotodama_b200 import train as train_mod
    from kotodama_b200.config import default_args
    from kotodama_b200.engine import TrainEngine
    real = TrainEngine.train_step
    calls = {"n": 0}

    def poisoned(self, micro, **kw):
        res = real(self, micro, **kw)
        calls["n"] += 1
        if calls["n"] == 3:
            res["loss"] = res["loss"] * float("nan")
        return res
    monkeypatch.setattr(TrainEngine, "train_step", poisoned)
    args = default_args(model_size="tiny", device="cpu", dtype="fp32", random_data=True, total_steps=6, sequence_length=32,
                        micro_batch_size=2, global_batch_tokens=64, checkpoint_dir=str(tmp_path), save_every=0,
                        log_every=100, warmup_steps=2, attn_res=True, attn_res_n_blocks=2, halt_on_nonfinite=True)
    with pytest.raises(RuntimeError, match="non-finite"):
        train_mod.train(args)
    assert calls["n"] == 3
    calls["n"] = 0
    args.halt_on_nonfinite = False                     # the reference's behaviour: log and continue
    out = train_mod.train(args)
    assert out["last_step"] == 5
