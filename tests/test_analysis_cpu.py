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
    tq = json.loads((out / "t" / "text_quality.json").read_text())["overall"]
    assert tq["n"] >= 1
    for fam, key in (("lexical", "yules_k"), ("coherence", "novelty_trend"), ("structural", "structural_variety_entropy"),
                     ("repetition", "repetition_onset_5gram"), ("creativity", "fabrication_density")):
        assert key in tq[fam]

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
    run("generate_report.py", "t", "--output-dir", out, "--metrics", mj)
    html = (out / "t" / "report.html").read_text()
    assert "Concept geometry" in html and "Activation geometry" in html and "Generations" in html
    assert "Training curves" in html and html.count("<svg") >= 4 and 'class="card"' in html


def test_text_quality_metrics_on_known_text(tmp_path):
    """The metric families on texts whose answer is known: a looping text, a varied text, two runs compared."""
    varied = ("Once upon a time there was a fox named Rune. He said, \"I will cross the river tomorrow.\" However, the river "
              "was wide because the rains of 1987 had come early. Did he cross it? He did! According to Dr. Hale, 45% of foxes never try.")
    looping = "the fox ran and ran and " * 12
    for name, texts in (("a", [varied, looping]), ("b", [looping, looping])):
        (tmp_path / name).mkdir()
        (tmp_path / name / "generations.json").write_text(json.dumps(
            {"run": name, "generations": [{"prompt": "p", "samples": texts}]}))
    sys.path.insert(0, str(TOOLS))
    import analyze_text_quality as tq
    v, l = tq.analyse(varied), tq.analyse(looping)
    assert l["repetition"]["loop_period"] == 6 and v["repetition"]["loop_period"] == 0
    assert l["repetition"]["repetition_onset_5gram"] >= 0 and v["repetition"]["repetition_onset_5gram"] == -1
    assert v["lexical"]["ttr_all"] > l["lexical"]["ttr_all"] and v["lexical"]["yules_k"] < l["lexical"]["yules_k"]
    assert v["structural"]["pct_interrogative"] > 0 and v["structural"]["pct_exclamatory"] > 0
    assert v["creativity"]["fabrication_density"] > 0 and v["creativity"]["quote_count"] == 1 and v["coherence"]["entity_count"] >= 2
    out = run("analyze_text_quality.py", "--input", tmp_path / "a" / "generations.json", tmp_path / "b" / "generations.json",
              "--output", tmp_path / "cmp", "--csv")
    cmp_ = json.loads((tmp_path / "cmp" / "text_quality_comparison.json").read_text())
    assert set(cmp_["profiles"]) == {"a", "b"} and cmp_["profiles"]["b"]["loop_rate"] == 1.0
    assert cmp_["most_distinctive"]["a"] and (tmp_path / "cmp" / "text_quality_profiles.csv").exists()
    assert "loop_rate" in out
