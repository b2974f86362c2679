"""Shared helpers of the analysis scripts: repository path, checkpoint selection, tokenizer, IO."""
from __future__ import annotations

import json
import sys
from pathlib import Path
from typing import Any, Optional

ROOT = Path(__file__).resolve().parents[2]
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

import torch  # noqa: E402
import yaml  # noqa: E402

from kotodama_b200.eval import load_checkpoint_registry, load_model  # noqa: E402
from kotodama_b200.data.tokenizer import load_tokenizer  # noqa: E402


def add_checkpoint_args(ap) -> None:
    ap.add_argument("--checkpoint", default=None, help="path of one checkpoint (.pt / .pt.zst)")
    ap.add_argument("--name", default=None, help="run name for --checkpoint")
    ap.add_argument("--checkpoints", default=None, help="comma-separated names from the registry")
    ap.add_argument("--registry", default=str(ROOT / "configs" / "checkpoints.yaml"))
    ap.add_argument("--section", "--config-section", dest="section", default="proxy", help="model section of the model YAML")
    ap.add_argument("--config", default=None, help="model YAML with named sections (default: the built-in size presets)")
    ap.add_argument("--attn-res", default=None, help="explicit AttnRes settings for --checkpoint: 'n_blocks=7' or 'boundaries=0,3,7,12'")
    ap.add_argument("--device", default="cpu")
    ap.add_argument("--output-dir", default="analysis")
    ap.add_argument("--tokenizer", default="HuggingFaceTB/SmolLM2-135M")


def parse_attn_res(spec: Optional[str]) -> Optional[dict[str, Any]]:
    """``'n_blocks=7'`` or ``'boundaries=0,3,7,12'`` -> the loader's explicit AttnRes settings."""
    if not spec:
        return None
    key, _, val = spec.partition("=")
    if key.strip() == "n_blocks":
        return {"attn_res": True, "attn_res_n_blocks": int(val)}
    if key.strip() == "boundaries":
        return {"attn_res": True, "attn_res_boundaries": [int(v) for v in val.split(",") if v.strip()]}
    raise SystemExit(f"--attn-res: expected 'n_blocks=N' or 'boundaries=a,b,c', got {spec!r}")


def select_checkpoints(args) -> list[tuple[str, dict[str, Any]]]:
    """[(run name, load_model kwargs)] from --checkpoint/--name or --checkpoints (registry)."""
    shared = {"config_path": args.config} if getattr(args, "config", None) else {}
    if args.checkpoint:
        return [(args.name or Path(args.checkpoint).stem,
                 dict(checkpoint=args.checkpoint, section=args.section, attn_res_config=parse_attn_res(getattr(args, "attn_res", None)),
                      **shared))]
    reg = load_checkpoint_registry(args.registry)
    names = [n.strip() for n in args.checkpoints.split(",")] if args.checkpoints else list(reg)
    out = []
    for n in names:
        if n not in reg:
            raise SystemExit(f"unknown checkpoint '{n}'; registry has {sorted(reg)}")
        info = reg[n]
        out.append((n, dict(checkpoint=info.path, section=info.model_section, attn_res_config=info.attn_res_config, **shared)))
    return out


def open_model(kw: dict[str, Any], device: str):
    dtype = torch.bfloat16 if str(device).startswith("cuda") else None
    return load_model(device=device, dtype=dtype, **kw)


def tokenizer(name: str):
    return load_tokenizer(name)


def run_dir(output_dir: str, run: str, track: Optional[str] = None) -> Path:
    d = Path(output_dir) / run / track if track else Path(output_dir) / run
    d.mkdir(parents=True, exist_ok=True)
    return d


def write_json(path: Path, obj: Any) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    with open(path, "w") as fh:
        json.dump(obj, fh, indent=1, default=lambda o: o.tolist() if hasattr(o, "tolist") else str(o))


def load_yaml(path: str | Path) -> Any:
    with open(path) as fh:
        return yaml.safe_load(fh)
