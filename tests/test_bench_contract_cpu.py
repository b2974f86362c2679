"""What the benchmark entry point promises that can be checked without a GPU: its reference arm, its flags, and the
clock sampler it runs beside the timed region."""
import json
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parents[1]


def test_reference_arm_reports_unavailable_and_exits_cleanly():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--impl", "reference", "--gpus", "1", "--steps", "2", "--warmup", "3"],
                       capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0, r.stderr[-1500:]
    lines = [l for l in r.stdout.splitlines() if l.startswith("{")]
    assert len(lines) == 1
    rec = json.loads(lines[0])
    assert rec["impl"] == "reference" and isinstance(rec["unavailable"], str) and "\n" not in rec["unavailable"]


def test_flags_of_the_contract_exist():
    r = subprocess.run([sys.executable, str(ROOT / "bench.py"), "--help"], capture_output=True, text=True, cwd=ROOT, timeout=300)
    assert r.returncode == 0
    for flag in ("--gpus", "--steps", "--warmup", "--impl", "--mode", "--model", "--fp8", "--micro-batch"):
        assert flag in r.stdout, flag
    src = (ROOT / "bench.py").read_text()
    for key in ('"metric"', '"value"', '"unit"', '"n_gpus"', '"ms_per_step"', '"higher_is_better"', '"scaling"', '"vs_baseline"',
                '"dtype"', '"data"', '"config"', '"clocks"', '"e2e"', '"gpu_launches"', '"h2d_bytes_per_step"', '"d2h_bytes_per_step"'):
        assert key in src, key
    assert "pin_memory" in src or "pinned" in src            # the end-to-end arm copies its inputs from pinned host memory
