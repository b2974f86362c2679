"""Data-parallel semantics on CPU ranks (gloo): loss decreases on a fixed batch, ranks end with
identical parameters, and two ranks equal one rank accumulating both batches."""
import json
import os
import subprocess
import sys

import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _launch(mode, out, nproc=2, steps=3, timeout=900):
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", OMP_NUM_THREADS="2")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(29600 + os.getpid() % 300),
           os.path.join(ROOT, "tests", "dist_worker.py"), "--mode", mode, "--out", out, "--steps", str(steps)]
    r = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert r.returncode == 0, r.stderr[-3000:]
    return [json.load(open(f"{out}.{mode}.{k}.json")) for k in range(nproc)]


def test_gloo_ddp_tiny_ranks_match_and_learn(tmp_path):
    res = _launch("cpu_ddp", str(tmp_path / "r"), steps=6)
    assert all(r["ranks_match"] for r in res)
    assert res[0]["checksum"] == res[1]["checksum"]
    for r in res:
        assert r["losses"][-1] < r["losses"][0] - 1.0, r["losses"]
    assert res[0]["momentum_entries"] == 28          # every Muon matrix, gathered from its owner


def test_two_ranks_equal_one_rank_with_accumulation(tmp_path):
    from kotodama_b200.config import MODEL_PRESETS, ModelConfig
    from kotodama_b200.engine import TrainEngine
    from kotodama_b200.models.llama import KotodamaModel
    res = _launch("cpu_ddp", str(tmp_path / "r"), steps=2)
    cfg = ModelConfig(**MODEL_PRESETS["tiny"], attn_res=True, attn_res_n_blocks=2)
    torch.manual_seed(0)
    eng = TrainEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32, muon_lr=0.02, adamw_lr=1e-3)
    batches = [torch.randint(0, cfg.vocab_size, (2, 256), generator=torch.Generator().manual_seed(100 + r))
               for r in range(2)]
    for _ in range(2):
        eng.train_step(batches)
    single = float(eng.arena.params.double().abs().sum())
    assert abs(single - res[0]["checksum"]) / single < 2e-4, (single, res[0]["checksum"])


def _single_process_reference(steps):
    from kotodama_b200.config import MODEL_PRESETS, ModelConfig
    from kotodama_b200.engine import TrainEngine
    from kotodama_b200.models.llama import KotodamaModel
    cfg = ModelConfig(**MODEL_PRESETS["smoke"], attn_res=True, attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    eng = TrainEngine(model, device="cpu", dtype=torch.float32, muon_lr=0.02, adamw_lr=1e-3)
    shared = torch.randint(0, cfg.vocab_size, (2, 64), generator=torch.Generator().manual_seed(7))
    losses = [float(eng.train_step([shared])["loss"]) for _ in range(steps)]
    return losses, float(sum(v.double().abs().sum() for v in model.state_dict().values()))


def test_tensor_parallel_with_sequence_parallel_matches_single_process(tmp_path):
    res = _launch("cpu_tp_sp", str(tmp_path / "r"), steps=3)
    losses, checksum = _single_process_reference(3)
    assert res[0]["q_shape"] == [256, 256] and res[0]["local_q_shape"] == [128, 256]
    assert res[0]["momentum_shape"] == [256, 256]
    for a, b in zip(res[0]["losses"], losses):
        assert abs(a - b) < 2e-3, (res[0]["losses"], losses)
    assert abs(res[0]["checksum"] - checksum) / checksum < 5e-4
    assert res[0]["checksum"] == res[1]["checksum"]


def test_tensor_parallel_allreduce_mode_and_autograd_api(tmp_path):
    losses, checksum = _single_process_reference(2)
    for mode in ("cpu_tp", "cpu_tp_autograd"):
        res = _launch(mode, str(tmp_path / mode), steps=2)
        for a, b in zip(res[0]["losses"], losses):
            assert abs(a - b) < 2e-3, (mode, res[0]["losses"], losses)
        assert abs(res[0]["checksum"] - checksum) / checksum < 5e-4, mode


def test_autograd_tp_api_matches_the_reference_tensor_parallel_code(tmp_path):
    """Two gloo ranks run the reference's unmodified tensor_parallel.py and this package's API side by side on the
    same weights: identical shards, the same loss, the same local gradients and the same clipped norm."""
    import pytest
    res = _launch("cpu_tp_reference_parity", str(tmp_path / "p"))
    if "skipped" in res[0]:
        pytest.skip(res[0]["skipped"])
    for r in res:
        assert r["shards_equal"] and r["local_q_rows"] == 32
        assert abs(r["loss_theirs"] - r["loss_ours"]) < 1e-5
        assert r["grad_rel_err_max"] < 1e-4, r
        assert abs(r["norm_theirs"] - r["norm_ours"]) / r["norm_theirs"] < 1e-4
    assert abs(res[0]["loss_ours"] - res[1]["loss_ours"]) < 1e-6


def test_tensor_parallel_serving_matches_single_process(tmp_path):
    """TP=2 serving over gloo: sharded heads / KV cache / MLP, all-reduced row projections, leader and
    follower in lock-step - same greedy tokens as the unsharded engine (fp32)."""
    res = _launch("cpu_tp_serve", str(tmp_path / "s"))
    for r in res:
        assert r["ranks_equal"]
        assert r["tp"] == r["ref"], (r["tp"], r["ref"])
        assert r["logit_rel_err_max"] < 1e-4 and r["logits_compared"] == 30
        # a request cancelled on the leader leaves every rank at the same step
        assert r["extra_equal"] and r["extra"][1][1] == "cancelled" and len(r["extra"][1][0]) < 5
        assert len(r["extra"][0][0]) == 5 and len(r["extra"][2][0]) == 5
        assert r["local_heads"] == 2 and r["local_kv"] == 1
        assert r["library_calls"] > 0 and r["native_calls"] == 0
    # steady-state steps carry a 32-byte header only: bodies were sent for the two admission steps and the cancel
    assert res[0]["control_steps"] > 8 and 0 < res[0]["control_body_bytes"] < 4000


def test_rank_leaves_between_steps_is_noticed_on_the_host(tmp_path):
    """One rank announces its departure between steps; the survivor raises PeerLeft before entering
    the next step (no collective is attempted, nothing waits for a timeout)."""
    res = _launch("cpu_rank_leaves", str(tmp_path / "h"), timeout=300)
    assert res[1]["outcome"] == "left" and res[1]["steps_done"] == 2
    assert res[0]["outcome"].startswith("peer_left") and "[1]" in res[0]["outcome"]
    assert res[0]["steps_done"] == 2


def test_rank_leaves_silently_ends_the_next_collective_with_an_error(tmp_path):
    """Without a notice the survivor's next collective fails within the process group's (short)
    timeout instead of hanging."""
    res = _launch("cpu_rank_leaves_silent", str(tmp_path / "s"), timeout=300)
    assert res[1]["outcome"] == "left"
    assert res[0]["outcome"].startswith("collective_error"), res[0]
    assert res[0]["detect_s"] < 60


def test_tensor_parallel_groups_replicated_data_parallel(tmp_path):
    """Four CPU ranks as two tensor-parallel groups of two, each group a data-parallel replica with its
    own batch: every rank ends with the same full parameters, equal to one process that takes both
    batches as micro-batches of one step."""
    res = _launch("cpu_tp2_dp2", str(tmp_path / "h"), nproc=4, steps=2)
    assert sorted((r["dp_rank"], r["tp_rank"]) for r in res) == [(0, 0), (0, 1), (1, 0), (1, 1)]
    assert all(r["replicas_match"] for r in res)
    r0 = res[0]
    assert r0["rel_param_diff"] < 5e-4, r0
    # a replica's loss is over its own batch; the mean over replicas is the one-process loss
    by_dp = {r["dp_rank"]: r["losses"] for r in res if r["tp_rank"] == 0}
    for i, ref in enumerate(r0["ref_losses"]):
        assert abs((by_dp[0][i] + by_dp[1][i]) / 2 - ref) < 2e-3, (by_dp, r0["ref_losses"])
