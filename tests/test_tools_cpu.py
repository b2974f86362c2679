"""The command-line tools under tools/ on small inputs, CPU only."""
import json
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parents[1]
sys.path.insert(0, str(ROOT / "tools"))


def tool(name, *args, timeout=600):
    r = subprocess.run([sys.executable, str(ROOT / "tools" / name), *map(str, args)], capture_output=True, text=True, cwd=ROOT,
                       timeout=timeout)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def write_metrics(path: Path, offset: float) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as fh:
        for s in range(0, 1000, 10):
            fh.write(json.dumps({"step": s, "train/loss": 5.0 - 0.002 * s + offset, "perf/tokens_per_sec": 1000.0}) + "\n")


def test_pull_metrics_local_runs_and_remote_copy(tmp_path):
    write_metrics(tmp_path / "run-a" / "metrics.jsonl", 0.0)
    write_metrics(tmp_path / "run-b" / "metrics.jsonl", 0.3)
    out = tool("pull_metrics.py", tmp_path / "run-a", tmp_path / "run-b", "--dynamics")
    lines = [json.loads(l) for l in out.splitlines() if l.startswith("{")]
    summ = {l["run"]: l for l in lines if "loss_final" in l}
    assert abs(summ["run-a"]["loss_final"] - 3.02) < 1e-9 and abs(summ["run-b"]["loss_final"] - 3.32) < 1e-9
    assert any("dynamics" in l for l in lines)
    rank = next(l for l in lines if "ranking" in l)
    assert rank["ranking"] == ["run-a", "run-b"] and abs(rank["loss_final_delta"]["run-b"] - 0.3) < 1e-9
    # the remote copy, with a stand-in for scp that serves one of the two files
    import pull_metrics

    class Done:
        def __init__(self, rc, err=""):
            self.returncode, self.stderr = rc, err
    calls = []

    def fake_scp(argv, **kw):
        calls.append(argv)
        src, dst = argv[-2], argv[-1]
        if src.endswith("/metrics.jsonl"):
            Path(dst).write_text((tmp_path / "run-a" / "metrics.jsonl").read_text())
            return Done(0)
        return Done(1, "scp: geo_metrics.jsonl: No such file or directory")
    got = pull_metrics.pull_remote("node7:~/ckpt/run-a/", tmp_path / "pulled", "scp", runner=fake_scp)
    assert [p.name for p in got] == ["metrics.jsonl"] and len(calls) == 2 and calls[0][0] == "scp"
    assert calls[0][-2] == "node7:~/ckpt/run-a/metrics.jsonl"
    assert pull_metrics.human(3 * 1024 * 1024) == "3.0 MB" and pull_metrics.metrics_path(str(tmp_path / "pulled")).name == "metrics.jsonl"


def test_log_and_trace_summaries(tmp_path):
    log = tmp_path / "train.log"
    with open(log, "w") as fh:
        for s in range(20):
            fh.write(f"step={s} | loss={5 - 0.1 * s:.4f} | lr=1e-3 | tok/s={30000 + 100 * s} | tokens=1 | gpu_mem=41.5GB\n")
            fh.write(f"device-timed: 800.0 ms/step, {40000 + s} tok/s\n")
    rec = json.loads(tool("extract_benchmark_results.py", log).splitlines()[-1])
    assert rec["lines"] == 20 and rec["gpu_mem_gb_max"] == 41.5 and abs(rec["loss_last"] - 3.1) < 1e-9
    assert rec["tok_s_median"] == 31100.0 and rec["device_tok_s_median"] == 40011.0
    trace = tmp_path / "trace.json"
    trace.write_text(json.dumps({"traceEvents": [
        {"cat": "kernel", "name": "gemm_kernel", "dur": 3000}, {"cat": "kernel", "name": "gemm_kernel", "dur": 1000},
        {"cat": "kernel", "name": "attn_kernel", "dur": 2000}, {"cat": "cpu_op", "name": "aten::mm", "dur": 9999}]}))
    out = tool("parse_profile.py", trace)
    rows = [l.split() for l in out.splitlines()[1:]]
    assert rows[0][0] == "gemm_kernel" and rows[0][1] == "4.00" and rows[0][2] == "2" and rows[1][0] == "attn_kernel"
    assert "device time 6.00 ms over 2 kernels" in out and "aten::mm" in out.split("host op")[1]


@pytest.mark.parametrize("optimizer", ["muon", "adamw"])
def test_profile_step_runs_on_cpu(tmp_path, optimizer):
    out = tool("profile_step.py", "--model", "tiny", "--device", "cpu", "--seq", 48, "--micro_batch", 2, "--steps", 1,
               "--warmup_steps", 1, "--optimizer", optimizer, "--trace", tmp_path / "t.json")
    assert "FORWARD_BACKWARD" in out and "OPTIMIZER_STEP" in out and "== ops" in out and "attention_fwd" in out
    assert ("ns_iteration" in out or "newton" in out.lower()) == (optimizer == "muon")
    assert (tmp_path / "t.json").stat().st_size > 1000


def test_eval_via_server_against_a_live_server(tmp_path):
    """The client of track 3 against the real HTTP server (uvicorn in a thread, tiny CPU engine)."""
    import socket
    import threading
    import time

    import torch
    uvicorn = pytest.importorskip("uvicorn")
    from kotodama_b200.config import ModelConfig
    from kotodama_b200.models.llama import KotodamaModel
    from kotodama_b200.serve.app import ByteTokenizer, create_app
    from kotodama_b200.serve.engine import ServingEngine
    torch.manual_seed(0)
    cfg = ModelConfig(hidden_size=64, num_layers=2, num_attention_heads=2, num_kv_heads=1, head_dim=32, intermediate_size=96,
                      vocab_size=300, max_position_embeddings=128, attn_res=True, attn_res_n_blocks=2)
    eng = ServingEngine(KotodamaModel(cfg), device="cpu", dtype=torch.float32, max_batch=8, max_ctx=128)
    app = create_app(eng, ByteTokenizer(), model_name="tiny")
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        port = s.getsockname()[1]
    server = uvicorn.Server(uvicorn.Config(app, host="127.0.0.1", port=port, log_level="error"))
    th = threading.Thread(target=server.run, daemon=True)
    th.start()
    try:
        prompts = tmp_path / "prompts.yaml"
        prompts.write_text("mini:\n  - \"Once upon\"\n  - \"The river\"\n  - \"In 1987\"\n")
        r = subprocess.run([sys.executable, str(ROOT / "tools" / "analysis" / "eval_via_server.py"), "--url", f"http://127.0.0.1:{port}",
                            "--name", "live", "--prompt-set", "mini", "--prompts-file", str(prompts), "--n-samples", "2",
                            "--max-tokens", "6", "--temperature", "0", "--concurrency", "4", "--wait", "30",
                            "--output-dir", str(tmp_path / "analysis")], capture_output=True, text=True, cwd=ROOT, timeout=300)
        assert r.returncode == 0, r.stderr[-2000:]
        out = json.loads((tmp_path / "analysis" / "live" / "generations.json").read_text())
        assert out["server_info"]["attn_res"] is True and out["server_stats"]["failed"] == 0 and out["server_stats"]["requests"] == 6
        assert len(out["generations"]) == 3 and all(len(g["samples"]) == 2 for g in out["generations"])
        for g in out["generations"]:
            assert g["samples"][0] == g["samples"][1]                              # greedy
            assert all(1 <= q["completion_tokens"] <= 6 for q in g["requests"])    # max_new_tokens reached the server
        # a request the server refuses (prompt longer than the context) is reported, not retried forever
        prompts.write_text("mini:\n  - \"" + "x" * 300 + "\"\n")
        r = subprocess.run([sys.executable, str(ROOT / "tools" / "analysis" / "eval_via_server.py"), "--url", f"http://127.0.0.1:{port}",
                            "--name", "bad", "--prompt-set", "mini", "--prompts-file", str(prompts), "--n-samples", "1",
                            "--output-dir", str(tmp_path / "analysis")], capture_output=True, text=True, cwd=ROOT, timeout=120)
        assert r.returncode == 0 and "HTTP 400" in r.stdout
        bad = json.loads((tmp_path / "analysis" / "bad" / "generations.json").read_text())
        assert bad["server_stats"]["failed"] == 1 and bad["generations"][0]["requests"][0]["attempts"] == 1
    finally:
        server.should_exit = True
        th.join(timeout=20)
        app.state.worker.shutdown()


def test_visualize_nca_pictures_and_round_trip(tmp_path):
    """Rule pictures (grid, strip, space-time), the complexity histogram, and decoding a generated token file."""
    import struct
    out = tool("visualize_nca.py", "--n-rules", 2, "--grid", 16, "--steps", 12, "--complexity-batch", 6, "--output-dir", tmp_path / "viz")
    assert "complexity of 6 sampled rules" in out
    for name in ("rule00_grid.png", "rule00_strip.png", "rule00_spacetime.png", "rule01_grid.png", "complexity_histogram.png", "summary.txt"):
        assert (tmp_path / "viz" / name).exists(), name
    png = (tmp_path / "viz" / "rule00_spacetime.png").read_bytes()
    assert png[:8] == b"\x89PNG\r\n\x1a\n" and png[12:16] == b"IHDR"
    w, h = struct.unpack(">II", png[16:24])
    assert w > 12 * 2 and h > 16 * 2                                     # 12 time steps wide, groups x 16 cells high
    # tokens written by the generator decode back into the grids they came from
    import numpy as np
    import torch
    import visualize_nca as vn
    from kotodama_b200.nca.generator import NCAConfig, NCARule, simulate_trajectory, tokenize_trajectory
    cfg = NCAConfig(grid_size=16, num_steps=6)
    torch.manual_seed(0)
    rule = NCARule(cfg.d_state, cfg.n_groups, 3, 16, 2)
    traj = simulate_trajectory(rule, cfg.grid_size, cfg.d_state, cfg.n_groups, cfg.num_steps, cfg.burn_in, 1.0, 0.5, device="cpu",
                               generator=torch.Generator().manual_seed(0))
    toks = np.asarray(tokenize_trajectory(traj, cfg.d_state, cfg.patch_size), dtype=np.int64)
    grids = vn.decode_tokens(toks, cfg)
    assert grids.shape == (cfg.num_steps * cfg.n_groups, 16, 16)
    assert np.array_equal(grids.reshape(cfg.num_steps, cfg.n_groups, 16, 16), traj[0].cpu().numpy())


def test_smoke_test_tool_passes_on_cpu():
    out = tool("smoke_test.py", "--device", "cpu", "--steps", 12, timeout=900)
    assert "FAIL" not in out and ("ok" in out.lower() or "pass" in out.lower())


def test_benchmark_matrix_on_the_tiny_cpu_configuration(tmp_path):
    out = tool("benchmark_matrix.py", "matrix", "--config", "configs/tiny-cpu.yaml", "--gpus", 1, "--only", "native,adamw_only",
               "--steps", 6, "--skip-lines", 1, "--out", tmp_path / "bm", "--", "--log_every", 1, timeout=900)
    recs = [json.loads(l) for l in (tmp_path / "bm" / "results_summary.jsonl").read_text().splitlines()]
    assert [r["name"] for r in recs] == ["native", "adamw_only"] and all(r["exit_code"] == 0 for r in recs)
    assert all(r["tok_s_median"] > 0 and r["lines"] == 6 for r in recs) and "--adamw_only" in recs[1]["flags"]
    assert "--log_every 1" in recs[0]["flags"] and "vs first" in out and "1.00x" in out
    meta = json.loads((tmp_path / "bm" / "metadata.json").read_text())
    assert meta["mode"] == "matrix" and set(meta["runs"]) == {"native", "adamw_only"} and "torch_version" in meta
    # the canary mode, commands only
    dry = tool("benchmark_matrix.py", "canary", "--models", "3b,8b", "--gpus", 8, "--dry-run", "--out", tmp_path / "c", "--", "--fp8")
    assert "--nproc-per-node 8 --master-addr 127.0.0.1" in dry and "canary-3b.yaml" in dry and "canary-8b.yaml" in dry and "--fp8" in dry
    import benchmark_matrix as bm
    text = bm.estimates([{"name": "3b", "tok_s_median": 360000.0, "gpu_mem_gb_max": 120.0}])
    assert "50 B tokens ->   1.6 days" in text and "250 B tokens" in text


def test_run_sweep_runs_arms_skips_finished_ones_and_compares(tmp_path):
    import yaml
    import run_sweep
    assert run_sweep.flags_of({"muon_lr": 0.02, "attn_res": True, "fp8": False, "x": None}) == ["--muon_lr", "0.02", "--attn_res"]
    for f in sorted((ROOT / "configs" / "sweeps").glob("*.yaml")):          # the shipped sweeps parse and build commands
        dry = tool("run_sweep.py", f, "--gpus", 8, "--dry-run", "--out", tmp_path / f.stem)
        spec = yaml.safe_load(f.read_text())
        assert dry.count("--checkpoint_dir") == len(spec["experiments"]) and "--nproc-per-node 8" in dry
    sweep = tmp_path / "s.yaml"
    sweep.write_text(yaml.safe_dump({"base": str(ROOT / "configs" / "tiny-cpu.yaml"),
                                     "common": {"total_steps": 4, "log_every": 1, "save_every": 999999},
                                     "experiments": {"adamw": {"adamw_only": True}, "muon": {"muon_lr": 0.02}, "unused": {}}}))
    out = tool("run_sweep.py", sweep, "--gpus", 1, "--only", "adamw,muon", "--out", tmp_path / "o")
    assert "ranking on train/loss" in out and "unused" not in out
    summary = json.loads((tmp_path / "o" / "sweep_summary.json").read_text())
    assert [r["name"] for r in summary["arms"]] == ["adamw", "muon"] and summary["comparison"]["baseline"] == "adamw"
    assert all((tmp_path / "o" / n / "DONE").exists() and (tmp_path / "o" / n / "metrics.jsonl").exists() for n in ("adamw", "muon"))
    again = tool("run_sweep.py", sweep, "--gpus", 1, "--only", "adamw,muon", "--out", tmp_path / "o")
    assert again.count("already done, skipped") == 2
    r = subprocess.run([sys.executable, str(ROOT / "tools" / "run_sweep.py"), str(sweep), "--only", "nope"], capture_output=True, text=True)
    assert r.returncode != 0 and "unknown arms" in r.stderr


def test_attnres_step_bench_compares_the_formulations_on_cpu():
    r = subprocess.run([sys.executable, str(ROOT / "benchmarks" / "attnres_step_bench.py"), "--model", "tiny", "--device", "cpu",
                        "--seq", "64", "--micro_batch", "2", "--iters", "2", "--warmup", "1", "--json",
                        "--arms", "baseline,blocked,per_call,module,blocks=1"], capture_output=True, text=True, cwd=ROOT, timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    arms = json.loads(r.stdout.strip().splitlines()[-1])["arms"]
    assert list(arms) == ["baseline", "blocked", "per_call", "module", "blocks=1"]
    assert arms["blocked"]["blocked_groups"] > 0 and arms["per_call"]["blocked_groups"] == 0 and arms["baseline"]["overhead_pct"] == 0.0
    assert all(v["ms"] > 0 and v["tokens_per_s"] > 0 for v in arms.values())


def test_roofline_floors_follow_from_the_shapes(tmp_path):
    peaks = tmp_path / "p.json"
    peaks.write_text(json.dumps({"hbm_gbs": 6451.8, "bf16_tflops_sustained": 1418.9}))
    t = json.loads(tool("roofline.py", "train", "--model", "3b", "--micro_batch", 8, "--seq", 4096, "--peaks", peaks, "--json",
                        "--measured_ms", 840))
    by = {r["op"]: r for r in t["ops"]}
    n, proj = 8 * 4096, 28 * (2 * 3072 * 3072 + 2 * 3072 * 1024 + 3 * 3072 * 8192)
    assert by["projections (fwd, dgrad, wgrad)"]["flops"] == pytest.approx(6.0 * proj * n)
    assert by["attention forward"]["flops"] == pytest.approx(2 * 2 * 28 * 3072 * 2048 * n)
    assert t["floor_ms"] == pytest.approx(sum(r["ms"] for r in t["ops"])) and 0.5 < t["fraction_of_floor"] < 1.0
    t8 = json.loads(tool("roofline.py", "train", "--model", "3b", "--gpus", 8, "--peaks", peaks, "--json"))
    ns1, ns8 = by["Newton-Schulz"]["flops"], {r["op"]: r for r in t8["ops"]}["Newton-Schulz"]["flops"]
    assert ns8 == pytest.approx(ns1 / 8) and "dp gradient reduction + parameter publish" in t8["comm_floor_ms"]
    d = json.loads(tool("roofline.py", "decode", "--model", "3b", "--batch", 64, "--context", 1220, "--peaks", peaks, "--json"))
    kv = 2.0 * 64 * 1220 * 28 * 2 * 1024
    assert {r["op"]: r["bytes"] for r in d["ops"]}["kv cache"] == pytest.approx(kv) and 2.2 < d["floor_ms"] < 2.4
    d8 = json.loads(tool("roofline.py", "decode", "--tp", 8, "--peaks", peaks, "--json"))
    assert d8["floor_ms"] == pytest.approx(d["floor_ms"] / 8)
    nominal = tool("roofline.py", "decode", "--peaks", tmp_path / "missing.json")
    assert "MEASURED_PEAKS.json" in nominal or "nominal" in nominal
