"""The training driver end to end on CPU: tiny AttnRes-Llama, fixed batch, Muon+AdamW,
checkpoint, resume equivalence, SIGTERM checkpoint, log-line format."""
import os
import re
import signal

import torch

from kotodama_b200.config import default_args, parse_args
from kotodama_b200.train import train


def _args(tmp, **kw):
    base = dict(model_size="smoke", attn_res=True, attn_res_n_blocks=2, sequence_length=64, micro_batch_size=2,
                global_batch_tokens=256, total_steps=6, warmup_steps=2, random_data=True, fixed_batch=True,
                device="cpu", dtype="fp32", checkpoint_dir=str(tmp), save_every=3, log_every=1, muon_lr=0.02,
                adamw_lr=1e-3, z_loss_weight=1e-4)
    base.update(kw)
    return default_args(**base)


def test_loss_decreases_and_checkpoints_written(tmp_path, caplog):
    import logging
    caplog.set_level(logging.INFO)
    out = train(_args(tmp_path, total_steps=8))
    assert out["losses"][-1] < out["losses"][0] - 0.5
    files = sorted(p.name for p in tmp_path.glob("step_*.pt"))
    assert files == ["step_00000003.pt", "step_00000006.pt", "step_00000007.pt"]
    line = [r.getMessage() for r in caplog.records if r.getMessage().startswith("step=")][-1]
    assert re.search(r"step=\d+/\d+ \| loss=\d+\.\d{4} \| z_loss=\d+\.\d{6} \| grad_norm=\d+\.\d{3} \| muon_lr=\S+ \| "
                     r"adamw_lr=\S+ \| tok/s=\d+ \| it/s=\S+ \| tokens=\S+B \| gpu_mem=\S+GB", line), line
    ck = torch.load(tmp_path / "step_00000007.pt", weights_only=False)
    assert set(ck) >= {"step", "tokens_consumed", "model", "muon_optimizer", "adamw_optimizer", "scheduler", "data"}
    assert "layers.0.attn.q_proj.weight" in ck["model"] and "ns_coefficients" in ck["muon_optimizer"]
    assert ck["tokens_consumed"] == 8 * 256


def test_resume_matches_uninterrupted_run(tmp_path):
    full = train(_args(tmp_path / "a", total_steps=6, save_every=100))
    part = train(_args(tmp_path / "b", total_steps=6, save_every=3))       # writes step 3 (and the final one)
    for p in (tmp_path / "b").glob("step_0000000[45]*"):
        p.unlink()
    (tmp_path / "b" / "step_00000005.pt").unlink(missing_ok=True)
    resumed = train(_args(tmp_path / "b", total_steps=6, save_every=100))  # resumes from step 3
    assert resumed["last_step"] == 5 and len(resumed["losses"]) == 2
    assert abs(resumed["losses"][-1] - full["losses"][-1]) < 5e-3, (resumed["losses"], full["losses"])


def test_sigterm_saves_and_stops(tmp_path):
    args = _args(tmp_path, total_steps=50, save_every=1000)
    import threading
    threading.Timer(1.0, lambda: os.kill(os.getpid(), signal.SIGTERM)).start()
    out = train(args)
    assert out["last_step"] < 49
    assert (tmp_path / f"step_{out['last_step']:08d}.pt").exists()


def test_yaml_config_and_cli_override(tmp_path):
    cfg = tmp_path / "c.yaml"
    cfg.write_text("model_size: smoke\nsequence-length: 128\nmuon_lr: 0.01\nbogus_key: 1\nattn_res: true\n")
    a = parse_args(["--config", str(cfg), "--muon_lr", "0.5"])
    assert a.model_size == "smoke" and a.sequence_length == 128 and a.muon_lr == 0.5 and a.attn_res is True
    assert not hasattr(a, "bogus_key")


def test_every_shipped_trainer_configuration_parses_without_unknown_keys(caplog):
    import logging
    from pathlib import Path
    import yaml
    root = Path(__file__).resolve().parents[1] / "configs"
    not_trainer = {"model.yaml", "checkpoints.yaml", "concepts.yaml", "prompts.yaml"}     # read by the eval loader / analysis tracks
    seen = 0
    for f in sorted(root.glob("*.yaml")):
        if f.name in not_trainer:
            continue
        with caplog.at_level(logging.WARNING):
            caplog.clear()
            a = parse_args(["--config", str(f)])
        assert not [r for r in caplog.records if "Unknown keys" in r.getMessage()], (f.name, caplog.text)
        keys = yaml.safe_load(f.read_text())
        assert all(getattr(a, k.replace("-", "_")) == v for k, v in keys.items()), f.name
        seen += 1
    assert seen >= 10
    full = parse_args(["--config", str(root / "training.yaml")])
    assert full.total_tokens == 80_000_000_000 and full.global_batch_tokens == 2_097_152 and full.batch_ramp_initial == 0.25
