"""Evaluation helpers shared by analysis scripts: model/registry loading, forward passes that
expose per-layer states and attention weights, text generation, memmap perplexity and JSONL
metrics access.

API parity with the reference's ``src/eval`` package (``src/eval/__init__.py:7-32``):
``load_model``, ``load_model_config``, ``load_checkpoint_registry``, ``CheckpointInfo``,
``forward_with_states``, ``compute_attention_weights``, ``ForwardResult``, ``generate``,
``generate_text``, ``compute_perplexity``, ``load_metrics``, ``get_nearest_step``,
``extract_series``.  One deliberate difference: the AttnRes forward here resets the partial sum
at block boundaries exactly like the model does; the reference's analysis copy forgets that
reset (``src/eval/forward.py:199-201`` against ``src/model/llama.py:701-703``).
"""
from __future__ import annotations

import json
import logging
import math
from dataclasses import dataclass, field
from pathlib import Path
from typing import Any, Optional

import numpy as np
import torch
import torch.nn.functional as F

from ..ckpt.manager import clean_state_dict, load_checkpoint_file
from ..config import MODEL_PRESETS, ModelConfig
from ..models.llama import KotodamaModel, route_sources

logger = logging.getLogger(__name__)


# ------------------------------------------------------------------------------ loading
@dataclass
class CheckpointInfo:
    name: str
    path: str
    model_section: str = "proxy"
    attn_res: bool = False
    attn_res_boundaries: Optional[list[int]] = None
    description: str = ""
    extra: dict[str, Any] = field(default_factory=dict)
    attn_res_n_blocks: Optional[int] = None
    group: Optional[str] = None
    tags: list[str] = field(default_factory=list)

    @property
    def attn_res_config(self) -> Optional[dict[str, Any]]:
        """The entry's explicit AttnRes settings (what `load_model` takes as ``attn_res_config``), or None when the
        entry names none and the loader should look at the checkpoint's keys."""
        given = {k: v for k, v in (("attn_res", self.attn_res or None), ("attn_res_n_blocks", self.attn_res_n_blocks),
                                   ("attn_res_boundaries", self.attn_res_boundaries)) if v is not None}
        return given or None


def load_model_config(config_path: Optional[str | Path] = None, section: str = "proxy", **overrides: Any) -> ModelConfig:
    """Model description from a YAML file with named sections (``model`` / ``proxy`` / ``8b`` /
    ``intermediate``) or, without a file, from the built-in presets."""
    kw: dict[str, Any] = {}
    if config_path is not None and Path(config_path).exists():
        import yaml
        raw = yaml.safe_load(open(config_path)) or {}
        sec = raw.get(section, raw.get("model", {}))
        fields = ModelConfig.__dataclass_fields__
        kw = {k: v for k, v in sec.items() if k in fields}
    else:
        alias = {"model": "3b", "full": "3b"}
        kw = dict(MODEL_PRESETS[alias.get(section, section)])
    kw.update(overrides)
    return ModelConfig(**kw)


def load_checkpoint_registry(path: str | Path) -> dict[str, CheckpointInfo]:
    """Named checkpoints from a YAML file, in either of two layouts:

    * flat: ``checkpoints: {name: {path, model_section, attn_res, attn_res_n_blocks, attn_res_boundaries, description}}``;
    * grouped, the reference's (``src/eval/model_loader.py:68-106``): ``{group: {checkpoints: {name: {path, tags,
      attn_res, attn_res_n_blocks, attn_res_boundaries}}}}`` - the group name and the tags are kept on the entry.
    """
    import yaml
    with open(path) as fh:
        raw = yaml.safe_load(fh) or {}
    known = {"path", "model_section", "attn_res", "attn_res_n_blocks", "attn_res_boundaries", "description", "tags"}
    out: dict[str, CheckpointInfo] = {}

    def add(name: str, e: dict[str, Any], group: Optional[str]) -> None:
        out[name] = CheckpointInfo(name=name, path=e["path"], model_section=e.get("model_section", "proxy"),
                                   attn_res=bool(e.get("attn_res", False)), attn_res_boundaries=e.get("attn_res_boundaries"),
                                   attn_res_n_blocks=e.get("attn_res_n_blocks"), description=e.get("description", ""),
                                   group=group, tags=list(e.get("tags", [])),
                                   extra={k: v for k, v in e.items() if k not in known})
    grouped = [g for g, v in raw.items() if g != "checkpoints" and isinstance(v, dict) and isinstance(v.get("checkpoints"), dict)]
    for g in grouped:
        for name, e in raw[g]["checkpoints"].items():
            add(name, e, g)
    flat = raw.get("checkpoints") if isinstance(raw.get("checkpoints"), dict) else (None if grouped else raw)
    for name, e in (flat or {}).items():
        if isinstance(e, dict) and "path" in e:
            add(name, e, None)
    return out


def detect_attn_res(state_dict: dict[str, torch.Tensor]) -> bool:
    return any(k.endswith("attn_res_query") or k == "final_res_query" for k in state_dict)


def load_model(checkpoint: str | Path, config: Optional[ModelConfig] = None, device: str = "cpu",
               dtype: Optional[torch.dtype] = None, section: str = "proxy", config_path: Optional[str] = None,
               attn_res_boundaries: Optional[list[int]] = None,
               attn_res_config: Optional[dict[str, Any]] = None) -> tuple[KotodamaModel, dict[str, Any]]:
    """Load a checkpoint (``.pt`` / ``.pt.zst``) into a model.  AttnRes comes from ``attn_res_config`` when given
    (``attn_res``, ``attn_res_n_blocks``, ``attn_res_boundaries``; naming blocks or boundaries implies ``attn_res``),
    else it is detected from the checkpoint's keys with seven uniform blocks - the reference's order of precedence
    (``src/eval/model_loader.py:109-175``).  Wrapper prefixes (``_orig_mod.``, ``module.``) are stripped, loading is
    non-strict."""
    ckpt = load_checkpoint_file(Path(checkpoint), map_location="cpu")
    sd = clean_state_dict(ckpt.get("model", ckpt))
    if config is None:
        if attn_res_config:
            explicit = dict(attn_res_config)
            explicit.setdefault("attn_res", True)
            config = load_model_config(config_path, section, **explicit)
        else:
            config = load_model_config(config_path, section, attn_res=detect_attn_res(sd))
        if attn_res_boundaries is not None:
            config.attn_res_boundaries = list(attn_res_boundaries)
        emb = sd.get("embed_tokens.weight")
        if emb is not None:
            config.vocab_size = emb.shape[0]
    model = KotodamaModel(config)
    missing, unexpected = model.load_state_dict(sd, strict=False)
    if missing or unexpected:
        logger.warning("load_model: %d missing, %d unexpected keys", len(missing), len(unexpected))
    model = model.to(device)
    if dtype is not None:
        model = model.to(dtype)
    meta = {k: ckpt.get(k) for k in ("step", "tokens_consumed") if isinstance(ckpt, dict)}
    return model.eval(), meta


# ------------------------------------------------------------------------------ forward
@dataclass
class ForwardResult:
    logits: torch.Tensor
    states: list[torch.Tensor]                    # states[0] = embeddings, states[i+1] = after layer i
    attention: dict[int, torch.Tensor] = field(default_factory=dict)
    route_weights: dict[str, torch.Tensor] = field(default_factory=dict)
    attention_outputs: list[torch.Tensor] = field(default_factory=list)   # attention branch of layer i, before the residual add


@torch.no_grad()
def compute_attention_weights(layer: Any, x_normed: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor
                              ) -> torch.Tensor:
    """Causal attention probabilities ``[B, heads, T, T]`` of one layer for its normalised input."""
    q, k, _ = layer.attn.project_qkv(x_normed, rope_cos, rope_sin)
    g = q.shape[1] // k.shape[1]
    sc = (q.float() @ k.repeat_interleave(g, 1).float().transpose(-1, -2)) / math.sqrt(q.shape[-1])
    T = x_normed.shape[1]
    mask = torch.ones(T, T, dtype=torch.bool, device=x_normed.device).tril()
    return torch.softmax(sc.masked_fill(~mask, float("-inf")), -1)


@torch.no_grad()
def forward_with_states(model: KotodamaModel, input_ids: torch.Tensor, attention_layers: Optional[list[int]] = None,
                        capture_attention_outputs: bool = False,
                        attention_fn: Optional[Any] = None) -> ForwardResult:
    """One forward pass that keeps what the analysis tracks look at: the residual state after every layer,
    the attention probabilities of ``attention_layers``, the depth-routing weights and - on request - every
    layer's attention-branch output.  ``attention_fn(layer, probs)``: called with each wanted layer's
    probabilities instead of keeping them (all layers of a long batch do not fit in memory at once)."""
    m, cfg = model, model.config
    want = set(attention_layers or [])
    x = m.embed_tokens(input_ids)
    states, attn, routes = [x], {}, {}
    branch: list[torch.Tensor] = []

    def see(i: int, layer: Any, h: torch.Tensor) -> None:
        if i in want:
            w = compute_attention_weights(layer, h, m.rope_cos, m.rope_sin)
            if attention_fn is not None:
                attention_fn(i, w)
            else:
                attn[i] = w
    if not cfg.attn_res:
        for i, layer in enumerate(m.layers):
            h = layer.attn_norm(x)
            see(i, layer, h)
            a = layer.attn(h, m.rope_cos, m.rope_sin)
            if capture_attention_outputs:
                branch.append(a)
            x = x + a
            x = x + layer.ffn(layer.ffn_norm(x))
            states.append(x)
        xf = m.norm(x)
    else:
        def weights(srcs, q, norm):
            u = torch.stack(srcs, 0).float()
            r = torch.rsqrt(u.pow(2).mean(-1) + norm.eps)
            return torch.softmax((u * (q * norm.weight).float()).sum(-1) * r, 0)
        committed: list[torch.Tensor] = []
        partial: Optional[torch.Tensor] = x
        for i, layer in enumerate(m.layers):
            srcs = committed + [partial]
            routes[f"attn_{i}"] = weights(srcs, layer.attn_res_query, layer.attn_res_norm).mean(dim=(1, 2))
            h = route_sources(srcs, layer.attn_res_query, layer.attn_res_norm.weight, layer.attn_res_norm.eps)
            if i in m._attn_res_boundary_set:
                committed.append(partial)
                partial = None
            hn = layer.attn_norm(h)
            see(i, layer, hn)
            a = layer.attn(hn, m.rope_cos, m.rope_sin)
            if capture_attention_outputs:
                branch.append(a)
            partial = a if partial is None else partial + a
            srcs = committed + [partial]
            routes[f"mlp_{i}"] = weights(srcs, layer.mlp_res_query, layer.mlp_res_norm).mean(dim=(1, 2))
            h = route_sources(srcs, layer.mlp_res_query, layer.mlp_res_norm.weight, layer.mlp_res_norm.eps)
            partial = partial + layer.ffn(layer.ffn_norm(h))
            states.append(h)
        srcs = committed + [partial]
        routes["final"] = weights(srcs, m.final_res_query, m.final_res_norm).mean(dim=(1, 2))
        xf = m.norm(route_sources(srcs, m.final_res_query, m.final_res_norm.weight, m.final_res_norm.eps))
        states[-1] = xf
    return ForwardResult(F.linear(xf, m.get_lm_head_weight()), states, attn, routes, branch)


# ------------------------------------------------------------------------------ generation
def _top_p_filter(logits: torch.Tensor, top_p: float) -> torch.Tensor:
    srt, idx = torch.sort(logits, descending=True)
    probs = torch.softmax(srt, -1)
    remove = probs.cumsum(-1) - probs > top_p
    return torch.full_like(logits, float("-inf")).scatter(-1, idx, srt.masked_fill(remove, float("-inf")))


@torch.no_grad()
def generate(model: KotodamaModel, input_ids: torch.Tensor, max_new_tokens: int = 64, temperature: float = 0.8,
             top_k: int = 50, top_p: Optional[float] = 0.0, repetition_penalty: float = 1.0, eos_token_id: Optional[int] = None,
             use_cache: bool = True, eos_tokens: Optional[list[int]] = None, max_seq_len: Optional[int] = None) -> torch.Tensor:
    """Batch-1 autoregressive generation with the model's own KV cache; returns prompt + new tokens.  Sampling order:
    repetition penalty, temperature, top-k, top-p, multinomial (``temperature <= 0``: greedy).  Generation ends at
    ``eos_token_id`` or any of ``eos_tokens``, after ``max_new_tokens``, or at ``max_seq_len`` / the model's context.
    With ``top_k=0`` and no repetition penalty this is the reference's ``generate`` (``src/eval/generate.py:24-101``)."""
    ids = input_ids.clone()
    past = None
    cur = ids
    stop = set(eos_tokens or []) | ({eos_token_id} if eos_token_id is not None else set())
    limit = min(max_seq_len or model.config.max_position_embeddings, model.config.max_position_embeddings)
    top_p = top_p or 0.0
    for _ in range(max_new_tokens):
        if ids.shape[1] >= limit:
            break
        out = model(cur if use_cache else ids, use_cache=use_cache, past_kv=past)
        past = out.get("past_kv") if use_cache else None
        lg = out["logits"][:, -1].float()
        if repetition_penalty != 1.0:
            seen = ids[0].unique()
            v = lg[0, seen]
            lg[0, seen] = torch.where(v > 0, v / repetition_penalty, v * repetition_penalty)
        if temperature <= 0:
            nxt = lg.argmax(-1, keepdim=True)
        else:
            lg = lg / temperature
            if top_k > 0:
                kth = torch.topk(lg, min(top_k, lg.shape[-1])).values[..., -1:]
                lg = lg.masked_fill(lg < kth, float("-inf"))
            if 0 < top_p < 1:
                lg = _top_p_filter(lg, top_p)
            nxt = torch.multinomial(torch.softmax(lg, -1), 1)
        ids = torch.cat([ids, nxt], 1)
        cur = nxt
        if int(nxt) in stop:
            break
    return ids


def generate_text(model: KotodamaModel, tokenizer: Any, prompt: str, details: bool = False, **kw: Any) -> Any:
    """The continuation of ``prompt`` as text.  ``details=True``: a record with the continuation, the number of
    new tokens and what ended the sample (``eos``, ``max_tokens`` or ``context``), as the reference's
    ``generate_text`` returns (``src/eval/generate.py:105-186``)."""
    dev = next(model.parameters()).device
    ids = torch.tensor([tokenizer.encode(prompt)], device=dev)
    eos = getattr(tokenizer, "eos_token_id", None)
    out = generate(model, ids, eos_token_id=eos, **kw)
    new = out[0, ids.shape[1]:].tolist()
    text = tokenizer.decode(new, skip_special_tokens=True)
    if not details:
        return text
    stop = set(kw.get("eos_tokens") or []) | ({eos} if eos is not None else set())
    ctx = model.config.max_position_embeddings
    if new and new[-1] in stop:
        why = "eos"
    elif out.shape[1] >= min(kw.get("max_seq_len") or ctx, ctx):
        why = "context"
    else:
        why = "max_tokens"
    return {"prompt": prompt, "continuation": text, "n_tokens": len(new), "stopped_by": why}


# ------------------------------------------------------------------------------ perplexity
@torch.no_grad()
def compute_perplexity(model: KotodamaModel, data_path: str | Path, seq_len: int = 2048, max_tokens: int = 1_000_000,
                       batch_size: int = 4, device: Optional[str] = None) -> dict[str, float]:
    """Token-level perplexity over the head of a flat uint16 token file (non-overlapping windows)."""
    dev = torch.device(device) if device else next(model.parameters()).device
    data = np.memmap(data_path, dtype=np.uint16, mode="r")
    n_win = min(len(data), max_tokens) // seq_len
    if n_win == 0:
        raise ValueError(f"{data_path}: fewer than {seq_len} tokens")
    nll, count = 0.0, 0
    for s in range(0, n_win, batch_size):
        rows = [np.asarray(data[w * seq_len:(w + 1) * seq_len]).astype(np.int64) for w in range(s, min(n_win, s + batch_size))]
        ids = torch.from_numpy(np.stack(rows)).to(dev)
        logits = model(ids)["logits"].float()
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]), ids[:, 1:].reshape(-1), reduction="sum")
        nll += float(loss)
        count += ids[:, 1:].numel()
    mean = nll / max(count, 1)
    return {"loss": mean, "perplexity": math.exp(min(mean, 50)), "tokens": float(count)}


# ------------------------------------------------------------------------------ metrics IO
def load_metrics(path: str | Path, merge: bool = True) -> dict[int, dict[str, float]]:
    """JSONL metrics -> ``{step: {key: value}}``; records of one step are merged, malformed lines skipped."""
    path = Path(path)
    if not path.exists():
        raise FileNotFoundError(f"Metrics file not found: {path}")
    out: dict[int, dict[str, float]] = {}
    for line in open(path):
        line = line.strip()
        if not line:
            continue
        try:
            rec = json.loads(line)
        except json.JSONDecodeError:
            continue
        step = rec.pop("step", None)
        if step is None:
            continue
        rec.pop("timestamp", None)
        if merge and int(step) in out:
            out[int(step)].update(rec)
        else:
            out[int(step)] = dict(rec)
    return out


def get_nearest_step(data: dict[int, dict[str, float]], target: int, tolerance: int = 500) -> Optional[int]:
    if not data:
        return None
    if target in data:
        return target
    best = min(data, key=lambda s: abs(s - target))
    return best if abs(best - target) <= tolerance else None


def extract_series(data: dict[int, dict[str, float]], key: str) -> list[tuple[int, float]]:
    """``[(step, value), ...]`` in step order for the steps that carry ``key``."""
    return [(s, float(data[s][key])) for s in sorted(data) if key in data[s] and data[s][key] is not None]


def extract_keys_matching(data: dict[int, dict[str, float]], prefix: str) -> list[str]:
    return sorted({k for r in data.values() for k in r if k.startswith(prefix)})


def get_value(data: dict[int, dict[str, float]], step: int, key: str) -> Optional[float]:
    """The metric at exactly this step, or None (``src/eval/metrics_io.py:170`` of the reference)."""
    return data.get(step, {}).get(key)


def load_multiple(paths: dict[str, str | Path]) -> dict[str, dict[int, dict[str, float]]]:
    return {name: load_metrics(p) for name, p in paths.items() if Path(p).exists()}
