"""The analysis tracks (tools/analysis) end to end on a tiny random checkpoint, CPU only."""
import importlib.util
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
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
    run("extract_activation_geometry.py", *common, "--prompt-set", "standard", "--components", "all", "--topo-subsample", 200)
    ag = out / "t" / "activation_geometry"
    geo = json.loads((ag / "geometry.json").read_text())
    L, H = cfg.num_layers, cfg.num_attention_heads
    assert len(geo["eigenspectra"]) == L + 1 and len(geo["effective_rank"]["q_proj"]["participation_ratio"]) == L
    assert len(geo["head_entropy"]["mean_per_layer"]) == L and 0 < geo["trajectories"]["straightness"] <= 1.0
    assert all(v > 0 for v in geo["topo_clouds"]["twonn_dimension"].values())
    for f in ("point_clouds", "topo_clouds", "trajectories", "attention_weights", "attention_outputs", "head_entropy", "weight_spectra"):
        assert (ag / f"{f}.npz").exists(), f
    with np.load(ag / "head_entropy.npz") as z:
        assert z["entropy"].shape == (L, H) and (z["entropy"] >= 0).all()
    with np.load(ag / "point_clouds.npz") as z:
        assert set(z.files) == {f"layer_{i}" for i in range(-1, L)} and z["layer_0"].shape[1] == cfg.hidden_size
    # a second run from token data, then the cross-run alignment from the files of both
    torch.manual_seed(1)
    ckpt2 = tmp_path / "other.pt"
    torch.save({"step": 10, "tokens_consumed": 1000, "model": KotodamaModel(cfg).state_dict()}, ckpt2)
    np.random.RandomState(0).randint(0, 260, size=8 * 48).astype("<u2").tofile(tmp_path / "eval.bin")
    for name, ck in (("t", ckpt), ("u", ckpt2)):
        run("extract_activation_geometry.py", "--checkpoint", ck, "--name", name, "--output-dir", out, "--tokenizer", "bytes",
            "--section", "tiny", "--components", "point_clouds", "--eval-data", tmp_path / "eval.bin", "--n-seqs", 8, "--seq-len", 48)
    run("extract_activation_geometry.py", "--components", "procrustes", "--runs", "t,u", "--output-dir", out)
    dist = json.loads((out / "_pairs" / "procrustes.json").read_text())["t|u"]
    assert len(dist) == L + 1 and all(0.0 <= d <= 1.0 for d in dist)
    run("extract_activation_geometry.py", *common, "--prompt-set", "standard", "--components", "all", "--topo-subsample", 200)
    run("visualize_activation_geometry.py", "--runs", "t,u", "--output-dir", out)
    have_mpl = importlib.util.find_spec("matplotlib") is not None
    ext = "png" if have_mpl else "svg"
    for fig in ("rankme", "head_entropy_mean", "effective_rank_q_proj", "point_cloud_layer0", "head_entropy_map"):
        assert (ag / f"{fig}.{ext}").exists(), fig
    assert (out / "_pairs" / f"compare_point_cloud_spread.{ext}").exists() and (out / "_pairs" / f"procrustes.{ext}").exists()

    # track 6
    run("extract_concept_geometry.py", *common, "--concept-sets", "weekdays,digits")
    run("analyze_concept_geometry.py", "--input", out / "t" / "concept_geometry", "--n-perm", 20)
    ana = json.loads((out / "t" / "concept_geometry" / "analysis.json").read_text())
    assert ana["sets"]["weekdays"]["kind"] == "cyclic" and "best_layer" in ana["sets"]["weekdays"]
    run("visualize_concept_geometry.py", "--input", out / "t" / "concept_geometry")
    for fig in ("weekdays_pca2", "weekdays_depth", "digits_pca2", "overview"):
        assert (out / "t" / "concept_geometry" / f"{fig}.{ext}").exists(), fig

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


def test_concept_geometry_statistics_on_planted_structure(tmp_path):
    """Activations with a known shape: a circle, a line, a map, a shared pair direction - and noise as control."""
    import math
    rng = np.random.default_rng(0)
    D, L, T = 32, 3, 2
    basis = np.linalg.qr(rng.normal(size=(D, D)))[0]

    def embed(low):                                      # [items, k] -> [T, items, L, D]: layer 0 is noise, the others carry it
        n, k = low.shape
        x = np.zeros((T, n, L, D), dtype=np.float32)
        for t in range(T):
            x[t, :, 0] = rng.normal(size=(n, D))
            for l in (1, 2):
                x[t, :, l] = low @ basis[:k] * 5 + rng.normal(size=(n, D)) * 0.05
        return x
    ang = np.arange(12) / 12 * 2 * math.pi
    coords = np.stack([rng.uniform(25, 49, 20), rng.uniform(-124, -70, 20)], 1)
    pair_base = rng.normal(size=(6, 4))
    pairs = np.zeros((12, 5))
    pairs[0::2, :4], pairs[1::2, :4], pairs[1::2, 4] = pair_base, pair_base, 3.0      # b = a + one shared direction
    sets = {"ring": ("cyclic", embed(np.stack([np.cos(ang), np.sin(ang)], 1)), {}),
            "line": ("ordinal", embed(np.arange(10, dtype=float)[:, None] / 3), {}),
            "map": ("geographic", embed(np.stack([coords[:, 1], coords[:, 0]], 1) / 10), {"coordinates": coords.tolist()}),
            "pairs": ("paired", embed(pairs), {}),
            "noise": ("cyclic", rng.normal(size=(T, 9, L, D)).astype(np.float32), {})}
    d = tmp_path / "cg"
    d.mkdir()
    meta = {"run": "planted", "sets": {}}
    for name, (kind, acts, extra) in sets.items():
        np.savez_compressed(d / f"{name}.npz", acts=acts, pooled=acts, last_tok=acts, token_counts=np.ones(acts.shape[:2], dtype=np.int32))
        meta["sets"][name] = {"kind": kind, "tier": 1, "items": [str(i) for i in range(acts.shape[1])], **extra}
    (d / "meta.json").write_text(json.dumps(meta))
    run("analyze_concept_geometry.py", "--input", d, "--n-perm", 99)
    ana = json.loads((d / "analysis.json").read_text())["sets"]
    ring, line, geo, pr, noise = (ana[k] for k in ("ring", "line", "map", "pairs", "noise"))
    assert ring["best_layer"]["r"] > 0.9 and ring["best_layer"]["p"] <= 0.02 and ring["best_layer"]["layer"] in (1, 2)
    assert abs(abs(ring["per_layer"][1]["cyclic"]["winding"]) - 1.0) < 0.05 and ring["per_layer"][1]["cyclic"]["knn_overlap"] == 1.0
    assert ring["first_significant_layer"] == 1                              # layer 0 is noise
    assert line["best_layer"]["r"] > 0.95 and line["per_layer"][2]["ordinal"]["pc1_rank_correlation"] > 0.99
    assert line["per_layer"][2]["direction"]["mean_cosine"] > 0.9 and line["per_layer"][2]["direction"]["z"] > 5
    assert geo["best_layer"]["r"] > 0.9 and geo["per_layer"][1]["geographic"]["map_fit"] > 0.9
    assert pr["per_layer"][1]["paired"]["completion_accuracy"] == 1.0 and pr["per_layer"][1]["paired"]["mean_cosine"] > 0.9
    assert pr["per_layer"][0]["paired"]["completion_accuracy"] < 0.5
    assert noise["best_layer"]["r"] < 0.5 and noise["significant_layers"] <= 1
    assert ring["per_layer"][1]["smoothness_to_next"] > 0.9 > ring["per_layer"][0]["smoothness_to_next"]
    assert ring["per_layer"][1]["subspace"]["top2_variance"] > 0.95 and ring["per_layer"][1]["template"]["distance_agreement"] > 0.9


def test_builtin_plotting_layer_draws_well_formed_figures():
    """kotodama_b200/eval/plot_utils.py: SVG figures without matplotlib - well-formed, everything inside the canvas,
    gaps where data is missing, stable run colours."""
    import math
    import re
    import xml.etree.ElementTree as ET

    from kotodama_b200.eval import plot_utils as pu
    ns = "{http://www.w3.org/2000/svg}"

    def inside(svg):
        root = ET.fromstring(svg)
        w, h = float(root.get("width")), float(root.get("height"))
        for el in root.iter():
            for k in ("x", "x1", "x2", "cx"):
                if el.get(k) is not None:
                    assert -1 <= float(el.get(k)) <= w + 1, (el.tag, k, el.get(k))
            for k in ("y", "y1", "y2", "cy"):
                if el.get(k) is not None:
                    assert -1 <= float(el.get(k)) <= h + 1, (el.tag, k, el.get(k))
            if el.get("points"):
                for pt in el.get("points").split():
                    x, y = map(float, pt.split(","))
                    assert 0 <= x <= w and 0 <= y <= h
        return root
    line = pu.line_chart({"proxy-muon": [5, 4, 3.5, None, 3.2, 3.1], "other <run>": [5, 4.5, 4.2, 4.0, float("nan"), 3.9]},
                         title="loss & <tags>", xlabel="step", ylabel="loss", x=[0, 10, 20, 30, 40, 50], dashed=["other <run>"])
    root = inside(line)
    polys = root.findall(f"{ns}polyline")
    assert len(polys) == 3                                   # the first series breaks at the missing value, the second ends before its NaN
    assert "&lt;tags&gt;" in line and "stroke-dasharray" in line and pu.run_color("proxy-muon") in line
    first = [tuple(map(float, p.split(","))) for p in polys[0].get("points").split()]
    assert [x for x, _ in first] == sorted(x for x, _ in first) and first[0][1] < first[-1][1]     # falling values go down the page
    ring = [(math.cos(i), math.sin(i)) for i in range(7)]
    inside(pu.scatter(ring, labels=list("MTWTFSS"), connect="loop", title="weekdays"))
    sc = pu.scatter([(0, 0), (1, 1), (2, 0), (3, 1)], arrows=[(0, 1), (2, 3)], ghosts=[(0.1, 0.2), (1.2, 0.9), (2, 0.3), (3.1, 1.1)])
    assert inside(sc) is not None and sc.count("marker-end") == 2
    hm = inside(pu.heatmap([[i * j for j in range(12)] for i in range(6)], title="entropy", xlabel="head", ylabel="layer"))
    assert len([r for r in hm.findall(f"{ns}rect")]) >= 6 * 12 + 40
    inside(pu.bar_chart({"a": 1.0, "b": -0.5, "c": 2.0}, title="bars"))
    inside(pu.line_chart({"flat": [1.0, 1.0, 1.0]}))                      # degenerate ranges do not divide by zero
    inside(pu.line_chart({"empty": []}))
    assert pu.run_color("some-run") == pu.run_color("some-run") and re.fullmatch(r"#[0-9a-f]{6}", pu.sequential_color(0.37))
    assert pu.run_label("a-very-long-run-name-indeed").endswith("…") and pu.run_label("proxy-nca") == "NCA"
