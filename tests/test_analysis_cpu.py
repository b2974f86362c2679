"""The analysis tracks (tools/analysis) end to end on a tiny random checkpoint, CPU only."""
import json
import subprocess
import sys
from pathlib import Path

import torch

from kotodama_b200.config import MODEL_PRESETS, ModelConfig
from kotodama_b200.models.llama import KotodamaModel

ROOT = Path(__file__).resolve().parents[1]
TOOLS = ROOT / "tools" / "analysis"


def run(script, *args):
    r = subprocess.run([sys.executable, str(TOOLS / script), *map(str, args)], capture_output=True, text=True, cwd=ROOT,
                       timeout=600)
    assert r.returncode == 0, r.stderr[-2000:]
    return r.stdout


def test_analysis_pipeline(tmp_path):
    cfg = ModelConfig(**dict(MODEL_PRESETS["tiny"], vocab_size=260), attn_res=True, attn_res_n_blocks=2)
    torch.manual_seed(0)
    model = KotodamaModel(cfg)
    ckpt = tmp_path / "step_00000010.pt"
    torch.save({"step": 10, "tokens_consumed": 1000, "model": model.state_dict()}, ckpt)
    out = tmp_path / "analysis"
    common = ["--checkpoint", ckpt, "--name", "t", "--output-dir", out, "--tokenizer", "bytes", "--section", "tiny"]

    # track 1/2: metrics
    mj = tmp_path / "metrics.jsonl"
    with open(mj, "w") as fh:
        for s in range(0, 200, 10):
            fh.write(json.dumps({"step": s, "train/loss": 5.0 - s * 0.01, "train/grad_norm": 1.0, "geo/rankme/layer_0": 10 + s * 0.01}) + "\n")
    run("analyze_run.py", mj, "--full", "--output", out / "t" / "training.json")
    assert "summary" in json.loads((out / "t" / "training.json").read_text())

    # track 3 + 4
    run("eval_generate.py", *common, "--no-ppl", "--max-tokens", 12, "--n-samples", 2)
    gen = json.loads((out / "t" / "generations.json").read_text())
    assert len(gen["generations"]) == 8 and len(gen["generations"][0]["samples"]) == 2
    run("analyze_text_quality.py", "--input", out / "t" / "generations.json")
    assert json.loads((out / "t" / "text_quality.json").read_text())["overall"]["n"] >= 1

    # track 5
    run("extract_activation_geometry.py", *common, "--prompt-set", "standard",
        "--components", "point_clouds,eigenspectra,trajectories,attention,effective_rank")
    geo = json.loads((out / "t" / "activation_geometry" / "geometry.json").read_text())
    assert len(geo["eigenspectra"]) == cfg.num_layers + 1 and geo["effective_rank"]
    run("visualize_activation_geometry.py", "--run", "t", "--output-dir", out)

    # track 6
    run("extract_concept_geometry.py", *common, "--concept-sets", "weekdays,digits")
    run("analyze_concept_geometry.py", "--input", out / "t" / "concept_geometry", "--n-perm", 20)
    ana = json.loads((out / "t" / "concept_geometry" / "analysis.json").read_text())
    assert ana["sets"]["weekdays"]["kind"] == "cyclic" and "best_layer" in ana["sets"]["weekdays"]
    run("visualize_concept_geometry.py", "--input", out / "t" / "concept_geometry")

    # report
    run("generate_report.py", "t", "--output-dir", out)
    html = (out / "t" / "report.html").read_text()
    assert "Concept geometry" in html and "Activation geometry" in html and "Generations" in html
