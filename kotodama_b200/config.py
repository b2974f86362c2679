"""Model / training configuration: presets, the flag table and YAML merging.

Parity targets in the reference project: the model dataclass at
``src/model/llama.py:91-140``, the size presets at ``src/training/train.py:91-152``
and the 56-flag CLI with two-pass YAML defaults at ``src/training/train.py:947-1206``.

The flag surface is declared as data (``FLAG_TABLE``) so the parser, the YAML
validator and the docs are generated from one place.  Flags that select a
third-party kernel backend in the reference (``--use_liger``, ``--compile``,
``--attn_impl``) are accepted for config compatibility and ignored: there is one
native kernel path.
"""
from __future__ import annotations

import argparse
import logging
import math
from dataclasses import asdict, dataclass
from typing import Any, Optional, Sequence

logger = logging.getLogger(__name__)


@dataclass
class ModelConfig:
    """Architecture description (field names match ``LuxiaModelConfig``)."""

    hidden_size: int = 3072
    num_layers: int = 28
    num_attention_heads: int = 24
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 8192
    vocab_size: int = 49152
    max_position_embeddings: int = 4096
    rope_theta: float = 500000.0
    norm_eps: float = 1e-5
    qk_norm: bool = True
    tie_word_embeddings: bool = True
    z_loss_weight: float = 1e-5
    activation_checkpointing: bool = False
    use_liger: bool = False          # accepted, ignored (single native path)
    attn_impl: str = "auto"          # accepted, ignored (single native path)
    attn_res: bool = False
    attn_res_n_blocks: int = 7
    attn_res_boundaries: Optional[list[int]] = None

    @property
    def num_kv_groups(self) -> int:
        return self.num_attention_heads // self.num_kv_heads

    @property
    def q_dim(self) -> int:
        return self.num_attention_heads * self.head_dim

    @property
    def kv_dim(self) -> int:
        return self.num_kv_heads * self.head_dim

    def boundaries(self) -> list[int]:
        """Sorted AttnRes block-boundary layers (``llama.py:545-551``)."""
        if self.attn_res_boundaries is not None:
            return sorted(set(int(b) for b in self.attn_res_boundaries))
        block = math.ceil(self.num_layers / self.attn_res_n_blocks)
        return list(range(0, self.num_layers, block))

    def param_count(self) -> int:
        """Same estimate as the reference (AttnRes parameters not counted)."""
        d = self.hidden_size
        attn = 2 * d * self.q_dim + 2 * d * self.kv_dim
        mlp = 3 * d * self.intermediate_size
        per_layer = attn + mlp + 2 * d + (2 * self.head_dim if self.qk_norm else 0)
        total = self.vocab_size * d + self.num_layers * per_layer + d
        if not self.tie_word_embeddings:
            total += self.vocab_size * d
        return total

    def matmul_params(self) -> int:
        """Parameters that take part in a GEMM per token (incl. the LM head)."""
        d = self.hidden_size
        per_layer = 2 * d * self.q_dim + 2 * d * self.kv_dim + 3 * d * self.intermediate_size
        return self.num_layers * per_layer + self.vocab_size * d

    def flops_per_token(self, seq_len: int) -> float:
        """6*N_matmul plus causal attention (fwd 2 GEMMs, bwd 4+1 recompute not counted)."""
        attn = 6 * self.num_layers * self.q_dim * seq_len  # 12*L*H*hd*T/2 (causal)
        return 6.0 * self.matmul_params() + attn

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


_SHAPE_KEYS = ("hidden_size", "num_layers", "num_attention_heads", "num_kv_heads", "head_dim",
               "intermediate_size", "vocab_size", "max_position_embeddings")


def _shape(*vals: int) -> dict[str, int]:
    return dict(zip(_SHAPE_KEYS, vals))


MODEL_PRESETS: dict[str, dict[str, int]] = {
    "full": _shape(3072, 28, 24, 8, 128, 8192, 49152, 4096),
    "3b": _shape(3072, 28, 24, 8, 128, 8192, 49152, 4096),
    "8b": _shape(4096, 32, 32, 8, 128, 14336, 49152, 4096),
    "intermediate": _shape(1024, 28, 8, 4, 128, 2816, 49152, 4096),
    "proxy": _shape(512, 28, 4, 2, 128, 1408, 49152, 4096),
    "smoke": _shape(256, 4, 4, 2, 64, 512, 1024, 2048),
    # CPU/gloo end-to-end slice: 256 wide, 4 layers, vocab 49152, FFN 688.
    "tiny": _shape(256, 4, 4, 2, 64, 688, 49152, 2048),
}


def model_config_from_args(args: argparse.Namespace) -> ModelConfig:
    if args.model_size not in MODEL_PRESETS:
        raise ValueError(f"Unknown model size '{args.model_size}'. Choose from: {list(MODEL_PRESETS)}")
    kw: dict[str, Any] = dict(MODEL_PRESETS[args.model_size])
    kw.update(
        qk_norm=True,
        z_loss_weight=args.z_loss_weight,
        activation_checkpointing=args.activation_checkpointing,
        use_liger=getattr(args, "use_liger", False),
        attn_impl=getattr(args, "attn_impl", "auto"),
        attn_res=args.attn_res,
        attn_res_n_blocks=args.attn_res_n_blocks,
    )
    if args.attn_res_boundaries:
        b = args.attn_res_boundaries
        kw["attn_res_boundaries"] = [int(x) for x in b.split(",")] if isinstance(b, str) else [int(x) for x in b]
    return ModelConfig(**kw)


# (name, kwargs) — kwargs go to ``add_argument``.  "flag" means store_true.
def _f(name: str, default: Any = None, typ: Any = None, flag: bool = False, choices: Optional[Sequence] = None,
       help: str = "") -> tuple[str, dict[str, Any]]:
    kw: dict[str, Any] = {"help": help}
    if flag:
        kw["action"] = "store_true"
    else:
        kw["default"] = default
        kw["type"] = typ if typ is not None else (type(default) if default is not None else str)
        if choices is not None:
            kw["choices"] = list(choices)
    return name, kw


FLAG_TABLE: list[tuple[str, dict[str, Any]]] = [
    _f("config", None, str, help="YAML file with defaults; CLI flags win"),
    # model
    _f("model_size", "proxy", str, choices=list(MODEL_PRESETS), help="size preset"),
    _f("z_loss_weight", 1e-5), _f("activation_checkpointing", flag=True),
    # AttnRes
    _f("attn_res", flag=True, help="Block Attention Residuals"),
    _f("no_attn_res", flag=True, help="turn Block Attention Residuals off (overrides a config file that enables them)"),
    _f("attn_res_n_blocks", 7), _f("attn_res_boundaries", None, str, help="e.g. '0,3,7,12,21,25'"),
    # scale
    _f("total_tokens", 6_000_000_000), _f("total_steps", None, int),
    _f("sequence_length", 2048), _f("micro_batch_size", 8), _f("global_batch_tokens", 2_097_152),
    _f("gradient_clip", 1.0),
    _f("batch_ramp_initial", 1.0), _f("batch_ramp_pct", 0.0),
    # optimizer
    _f("adamw_only", flag=True),
    _f("muon_lr", 0.03), _f("muon_momentum", 0.95), _f("muon_weight_decay", 0.01),
    _f("muon_ns_iterations", 5),
    _f("muon_ns_coefficients", None, str, choices=["original", "gram_ns", "polar_express"]),
    _f("adamw_lr", 6e-4), _f("adamw_beta1", 0.9), _f("adamw_beta2", 0.95), _f("adamw_weight_decay", 0.1),
    # schedule
    _f("warmup_steps", 2000), _f("decay_start_pct", 0.90), _f("decay_type", "sqrt"),
    # data
    _f("data_path", ""), _f("random_data", flag=True), _f("seed", 42),
    # checkpoint
    _f("checkpoint_dir", "checkpoints"), _f("save_every", 1000), _f("keep_checkpoints", 5),
    _f("async_checkpoint", flag=True), _f("checkpoint_shm_dir", "/dev/shm/luxia-base-ckpts"),
    # logging / profiling / monitoring
    _f("log_every", 10),
    _f("profile", flag=True), _f("profile_start_step", 50), _f("profile_steps", 20), _f("profile_dir", None, str),
    _f("geo_monitor", flag=True), _f("geo_monitor_tier1_every", 500), _f("geo_monitor_tier2_every", 5000),
    # NCA transition
    _f("resume_nca", None, str), _f("reinit_mlps", flag=True),
    # precision / kernels (compat)
    _f("fp8", flag=True), _f("use_liger", flag=True),
    _f("attn_impl", "auto", str, choices=["auto", "fa2", "fa4", "sdpa"]),
    _f("compile", flag=True),
    # parallelism
    _f("tp_size", 1),
    # wandb
    _f("wandb", flag=True), _f("wandb_project", "luxia-base"), _f("wandb_run_name", None, str),
    # ---- additions of this framework ----
    _f("device", "cuda", str, choices=["cuda", "cpu"]),
    _f("backend", "auto", str, choices=["auto", "nccl", "gloo", "native"],
       help="'native' = in-kernel NVLink collectives; 'nccl'/'gloo' = library collectives"),
    _f("dtype", "bf16", str, choices=["bf16", "fp32"]),
    _f("sequence_parallel", flag=True),
    _f("distributed_muon", flag=True, help="each Muon matrix is orthogonalised by one owner rank (the default)"),
    _f("no_distributed_muon", flag=True, help="repeat Newton-Schulz on every rank, as the reference does"),
    _f("halt_on_nonfinite", flag=True, help="stop the run (all ranks) when the loss or gradient norm is not finite"),
    _f("watchdog_s", 0.0, float, help="log which rank and phase stalled when a step phase exceeds this many seconds (0: off)"),
    _f("fp8_recipe", "block128", str, choices=["tensorwise", "block128"]),
    _f("reference_lr_order", flag=True,
       help="apply the schedule after the optimizer step (step 0 at full LR, step 1 at LR 0)"),
    _f("fixed_batch", flag=True, help="repeat one batch per rank (learnability checks)"),
]


def build_parser() -> argparse.ArgumentParser:
    p = argparse.ArgumentParser(description="kotodama-b200 distributed training")
    for name, kw in FLAG_TABLE:
        p.add_argument(f"--{name}", **kw)
    p.add_argument("--checkpoint_compress", action="store_true", default=True)
    p.add_argument("--no_checkpoint_compress", dest="checkpoint_compress", action="store_false")
    return p


def load_yaml_defaults(path: str) -> dict[str, Any]:
    import yaml

    with open(path) as fh:
        raw = yaml.safe_load(fh) or {}
    return {str(k).replace("-", "_"): v for k, v in raw.items()}


def parse_args(argv: Optional[Sequence[str]] = None) -> argparse.Namespace:
    """Two-pass parse: YAML values become defaults, explicit CLI flags override them."""
    parser = build_parser()
    args = parser.parse_args(argv)
    if args.config is not None:
        cfg = load_yaml_defaults(args.config)
        known = {a.dest for a in parser._actions}
        unknown = sorted(set(cfg) - known)
        if unknown:
            logger.warning("Unknown keys in %s (ignored): %s", args.config, ", ".join(unknown))
        parser.set_defaults(**{k: v for k, v in cfg.items() if k in known})
        args = parser.parse_args(argv)
        args._config_file = args.config
    if getattr(args, "no_attn_res", False):
        args.attn_res = False
    return args


def default_args(**overrides: Any) -> argparse.Namespace:
    """Namespace with every flag at its default, for programmatic use."""
    ns = build_parser().parse_args([])
    for k, v in overrides.items():
        setattr(ns, k, v)
    return ns


def grad_accum_for_step(step: int, total_steps: int, base: int, initial_fraction: float, ramp_pct: float) -> int:
    """Linear batch-size ramp over the first ``ramp_pct`` of training (``train.py:853-878``)."""
    if ramp_pct <= 0 or initial_fraction >= 1.0:
        return base
    ramp_steps = int(total_steps * ramp_pct)
    if step >= ramp_steps:
        return base
    frac = initial_fraction + (1.0 - initial_fraction) * (step / max(ramp_steps, 1))
    return max(1, int(base * frac))
