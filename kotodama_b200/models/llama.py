"""Llama-family decoder with GQA, QK-norm, RoPE, SwiGLU, tied embeddings, z-loss and
Block Attention Residuals (AttnRes).

This module is the *definition* of the model: parameter names and registration order
are identical to the reference (``src/model/llama.py:446-581``) so that checkpoints
load both ways, and ``forward`` is a plain autograd implementation that runs on any
device.  It is the numerical oracle for the hand-scheduled training executor
(``kotodama_b200.engine``) and the serving engine, which run the same math through
sm_100a kernels.

AttnRes semantics (``llama.py:605-716``): every sub-layer input is a softmax-weighted
mixture over "sources" = committed block summaries (oldest first) + the running
partial sum of the current block.  Keys are RMS-normalised sources scaled by a
per-call learned weight, values are the raw sources, the pseudo-query is zero at
init (uniform average).  At a boundary layer the pre-attention route still sees the
old partial; the partial is then committed and restarted from zero.
"""
from __future__ import annotations

import math
from typing import Any, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import ModelConfig


class RMSNorm(nn.Module):
    """``x * rsqrt(mean(x^2) + eps) * weight`` in the input dtype (``llama.py:143-153``)."""

    def __init__(self, dim: int, eps: float = 1e-5) -> None:
        super().__init__()
        self.eps = eps
        self.weight = nn.Parameter(torch.ones(dim))

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + self.eps) * self.weight


def rope_tables(head_dim: int, max_pos: int, theta: float = 500000.0,
                device: Optional[torch.device] = None) -> tuple[torch.Tensor, torch.Tensor]:
    """cos/sin tables ``[max_pos, head_dim]`` with the half-tables duplicated (``llama.py:156-169``)."""
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, device=device).float() / head_dim))
    ang = torch.outer(torch.arange(max_pos, device=device).float(), inv)
    return torch.cat([ang.cos(), ang.cos()], -1), torch.cat([ang.sin(), ang.sin()], -1)


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seq_dim: int = 2) -> torch.Tensor:
    """Rotate-half RoPE.  ``seq_dim=2`` for (B,H,S,D), ``seq_dim=1`` for (B,S,H,D)."""
    shape = [1, 1, 1, x.shape[-1]]
    shape[seq_dim] = cos.shape[0]
    return x * cos.view(shape) + rotate_half(x) * sin.view(shape)


def apply_rope_fa2(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    return apply_rope(x, cos, sin, seq_dim=1)


class GQAttention(nn.Module):
    """Grouped-query attention; QK-norm (weight ``[head_dim]`` shared by heads) precedes RoPE."""

    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        self.num_heads = config.num_attention_heads
        self.num_kv_heads = config.num_kv_heads
        self.head_dim = config.head_dim
        self.num_kv_groups = config.num_kv_groups
        self.tp_group = None
        d = config.hidden_size
        self.q_proj = nn.Linear(d, self.num_heads * self.head_dim, bias=False)
        self.k_proj = nn.Linear(d, self.num_kv_heads * self.head_dim, bias=False)
        self.v_proj = nn.Linear(d, self.num_kv_heads * self.head_dim, bias=False)
        self.o_proj = nn.Linear(self.num_heads * self.head_dim, d, bias=False)
        self.qk_norm = config.qk_norm
        if self.qk_norm:
            self.q_norm = RMSNorm(self.head_dim, eps=config.norm_eps)
            self.k_norm = RMSNorm(self.head_dim, eps=config.norm_eps)

    def project_qkv(self, x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, pos_offset: int = 0
                    ) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """Post-norm, post-RoPE q/k and v in (B, heads, S, hd) layout."""
        b, s, _ = x.shape
        # Under tensor parallelism the projections hold a slice of the heads.
        q = self.q_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        k = self.k_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        v = self.v_proj(x).view(b, s, -1, self.head_dim).transpose(1, 2)
        if self.qk_norm:
            q, k = self.q_norm(q), self.k_norm(k)
        c, sn = cos[pos_offset:pos_offset + s], sin[pos_offset:pos_offset + s]
        return apply_rope(q, c, sn), apply_rope(k, c, sn), v

    def forward(self, x: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                mask: Optional[torch.Tensor] = None,
                past_kv: Optional[tuple[torch.Tensor, torch.Tensor]] = None,
                use_cache: bool = False) -> Any:
        if self.tp_group is not None:
            from ..parallel.tp import copy_to_parallel_region
            x = copy_to_parallel_region(x, self.tp_group)
        b, s, _ = x.shape
        pos = past_kv[0].shape[2] if past_kv is not None else 0
        q, k, v = self.project_qkv(x, rope_cos, rope_sin, pos)
        if past_kv is not None:
            k = torch.cat([past_kv[0], k], dim=2)
            v = torch.cat([past_kv[1], v], dim=2)
        new_kv = (k, v)
        out = F.scaled_dot_product_attention(
            q, k, v, attn_mask=mask, is_causal=(past_kv is None and mask is None and s > 1),
            enable_gqa=(q.shape[1] != k.shape[1]))
        out = self.o_proj(out.transpose(1, 2).reshape(b, s, -1))
        if self.tp_group is not None:
            from ..parallel.tp import reduce_from_parallel_region
            out = reduce_from_parallel_region(out, self.tp_group)
        return (out, new_kv) if use_cache else out


class SwiGLUFFN(nn.Module):
    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        self.gate_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.up_proj = nn.Linear(config.hidden_size, config.intermediate_size, bias=False)
        self.down_proj = nn.Linear(config.intermediate_size, config.hidden_size, bias=False)
        self.tp_group = None

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        if self.tp_group is not None:
            from ..parallel.tp import copy_to_parallel_region, reduce_from_parallel_region
            x = copy_to_parallel_region(x, self.tp_group)
        out = self.down_proj(F.silu(self.gate_proj(x)) * self.up_proj(x))
        if self.tp_group is not None:
            out = reduce_from_parallel_region(out, self.tp_group)
        return out


class TransformerBlock(nn.Module):
    """Pre-norm block.  Owns the two AttnRes pseudo-queries and key norms of its sub-layers."""

    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        if config.attn_res:  # direct parameters first: keeps the reference's named_parameters order
            self.attn_res_query = nn.Parameter(torch.zeros(config.hidden_size))
            self.mlp_res_query = nn.Parameter(torch.zeros(config.hidden_size))
        self.attn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.attn = GQAttention(config)
        self.ffn_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.ffn = SwiGLUFFN(config)
        if config.attn_res:
            self.attn_res_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
            self.mlp_res_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)

    def forward(self, x: torch.Tensor, rope_cos: torch.Tensor, rope_sin: torch.Tensor,
                mask: Optional[torch.Tensor] = None, past_kv: Any = None, use_cache: bool = False) -> Any:
        new_kv = None
        if use_cache:
            a, new_kv = self.attn(self.attn_norm(x), rope_cos, rope_sin, mask, past_kv, use_cache=True)
        else:
            a = self.attn(self.attn_norm(x), rope_cos, rope_sin, mask)
        x = x + a
        x = x + self.ffn(self.ffn_norm(x))
        return (x, new_kv) if use_cache else x


def route_sources(sources: list[torch.Tensor], query: torch.Tensor, norm_weight: torch.Tensor,
                  eps: float) -> torch.Tensor:
    """AttnRes routing over a list of active sources, statistics in fp32.

    ``r_j = rsqrt(mean(u_j^2)+eps)``, ``l_j = (u_j . (query*norm_weight)) r_j``,
    ``h = sum_j softmax(l)_j u_j`` (``llama.py:630-644``)."""
    buf = torch.stack(sources, 0)
    up = (lambda t: t) if buf.dtype == torch.float64 else (lambda t: t.float())
    w = up(query * norm_weight)
    bf = up(buf)
    r = torch.rsqrt(bf.pow(2).mean(-1) + eps)
    logits = (bf * w).sum(-1) * r
    alpha = torch.softmax(logits, 0)
    return (alpha.unsqueeze(-1) * bf).sum(0).to(buf.dtype)


def route_blocked(committed: list[torch.Tensor], partial: Optional[torch.Tensor], query: torch.Tensor,
                  norm_weight: torch.Tensor, eps: float) -> torch.Tensor:
    """Two-phase form of the same routing (``serve.py:113-164``): phase 1 over the committed
    blocks yields ``o`` and ``lse``; phase 2 merges the partial with ``pi = sigmoid(l_p - lse)``."""
    w = (query * norm_weight).float()
    c = torch.stack(committed, 0).float()
    r = torch.rsqrt(c.pow(2).mean(-1) + eps)
    logits = (c * w).sum(-1) * r
    lse = torch.logsumexp(logits, 0)
    o = (torch.softmax(logits, 0).unsqueeze(-1) * c).sum(0)
    if partial is None:
        return o.to(committed[0].dtype)
    p = partial.float()
    lp = (p * w).sum(-1) * torch.rsqrt(p.pow(2).mean(-1) + eps)
    pi = torch.sigmoid(lp - lse).unsqueeze(-1)
    return (o + pi * (p - o)).to(partial.dtype)


class KotodamaModel(nn.Module):
    """The decoder.  ``forward(input_ids, labels, mask, past_kv, use_cache)`` returns a dict with
    ``loss`` (cross-entropy **plus** z-loss), ``z_loss`` (already weighted), ``logits`` and
    ``past_kv`` as applicable (``llama.py:765-855``)."""

    def __init__(self, config: ModelConfig) -> None:
        super().__init__()
        self.config = config
        if config.attn_res:
            self.final_res_query = nn.Parameter(torch.zeros(config.hidden_size))
        self.embed_tokens = nn.Embedding(config.vocab_size, config.hidden_size)
        self.layers = nn.ModuleList([TransformerBlock(config) for _ in range(config.num_layers)])
        self.norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
        self.lm_head = None if config.tie_word_embeddings else nn.Linear(
            config.hidden_size, config.vocab_size, bias=False)
        if config.attn_res:
            self.final_res_norm = RMSNorm(config.hidden_size, eps=config.norm_eps)
            self._attn_res_boundary_set = frozenset(config.boundaries())
            self._attn_res_max_sources = len(self._attn_res_boundary_set) + 1
            masks = torch.zeros(2 * config.num_layers + 1, self._attn_res_max_sources, dtype=torch.bool)
            n = 0
            for i in range(config.num_layers):
                masks[2 * i, : n + 1] = True
                if i in self._attn_res_boundary_set:
                    n += 1
                masks[2 * i + 1, : n + 1] = True
            masks[2 * config.num_layers, : n + 1] = True
            self.register_buffer("_attn_res_masks", masks, persistent=False)
            self._attn_res_active_counts = [n for _, _, n in self.routing_table()]
        cos, sin = rope_tables(config.head_dim, config.max_position_embeddings, config.rope_theta)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)
        self._init_weights()

    def materialize_buffers(self, device: torch.device | str) -> None:
        """(Re)create the non-persistent buffers on ``device``; needed after meta-device construction."""
        c = self.config
        cos, sin = rope_tables(c.head_dim, c.max_position_embeddings, c.rope_theta, device=torch.device(device))
        self.rope_cos, self.rope_sin = cos, sin
        if c.attn_res:
            m = self._attn_res_masks
            if m.is_meta:
                masks = torch.zeros(2 * c.num_layers + 1, self._attn_res_max_sources, dtype=torch.bool)
                for j, (_, _, n) in enumerate(self.routing_table()):
                    masks[j, :n] = True
                m = masks
            self._attn_res_masks = m.to(device)

    # ---- initialisation -------------------------------------------------
    def _init_weights(self) -> None:
        std = 0.02
        for m in self.modules():
            if isinstance(m, (nn.Linear, nn.Embedding)):
                nn.init.normal_(m.weight, mean=0.0, std=std)
        scale = 1.0 / math.sqrt(2 * self.config.num_layers)
        for layer in self.layers:
            nn.init.normal_(layer.attn.o_proj.weight, mean=0.0, std=std * scale)
            nn.init.normal_(layer.ffn.down_proj.weight, mean=0.0, std=std * scale)

    def get_lm_head_weight(self) -> torch.Tensor:
        return self.lm_head.weight if self.lm_head is not None else self.embed_tokens.weight

    def reinit_mlps(self) -> None:
        """Fresh MLP weights after NCA pre-pre-training (``llama.py:857-864``)."""
        scale = 1.0 / math.sqrt(2 * self.config.num_layers)
        for layer in self.layers:
            nn.init.normal_(layer.ffn.gate_proj.weight, std=0.02)
            nn.init.normal_(layer.ffn.up_proj.weight, std=0.02)
            nn.init.normal_(layer.ffn.down_proj.weight, std=0.02 * scale)

    def reinit_embeddings(self, new_vocab_size: Optional[int] = None) -> None:
        """Fresh (optionally resized) embeddings when moving from the NCA vocabulary to language."""
        w = self.embed_tokens.weight
        if new_vocab_size is not None and new_vocab_size != self.config.vocab_size:
            self.config.vocab_size = new_vocab_size
            self.embed_tokens = nn.Embedding(new_vocab_size, self.config.hidden_size, device=w.device, dtype=w.dtype)
            if self.lm_head is not None:
                self.lm_head = nn.Linear(self.config.hidden_size, new_vocab_size, bias=False,
                                         device=w.device, dtype=w.dtype)
        nn.init.normal_(self.embed_tokens.weight, std=0.02)
        if self.lm_head is not None:
            nn.init.normal_(self.lm_head.weight, std=0.02)

    # ---- AttnRes --------------------------------------------------------
    @staticmethod
    def _route_static(buf: torch.Tensor, query: torch.Tensor, norm: nn.Module,
                      active_mask: torch.Tensor, num_active: int = 0) -> torch.Tensor:
        """Padded-buffer form used by monitors and analysis code: ``buf`` is (max_S, B, T, D)."""
        n = num_active or int(active_mask.sum())
        return route_sources(list(buf[:n].unbind(0)), query, norm.weight, norm.eps)

    def _block_attn_res_from_list(self, sources: list[torch.Tensor], query: torch.Tensor,
                                  norm: nn.Module) -> torch.Tensor:
        return route_sources(list(sources), query, norm.weight, norm.eps)

    def routing_table(self) -> list[tuple[str, int, int]]:
        """``(kind, layer, n_active_sources)`` for the 2L+1 routing calls, in execution order."""
        out: list[tuple[str, int, int]] = []
        n = 0
        for i in range(self.config.num_layers):
            out.append(("attn", i, n + 1))
            if i in self._attn_res_boundary_set:
                n += 1
            out.append(("mlp", i, n + 1))
        out.append(("final", self.config.num_layers, n + 1))
        return out

    def _forward_attn_res(self, embed: torch.Tensor, mask: Optional[torch.Tensor], past_kv: Any = None,
                          use_cache: bool = False, collect: Optional[list] = None) -> tuple[torch.Tensor, list]:
        committed: list[torch.Tensor] = []
        partial: Optional[torch.Tensor] = embed
        new_kv: list = []
        for i, layer in enumerate(self.layers):
            srcs = committed + ([partial] if partial is not None else [])
            h = route_sources(srcs, layer.attn_res_query, layer.attn_res_norm.weight, layer.attn_res_norm.eps)
            if i in self._attn_res_boundary_set:
                committed.append(partial if partial is not None else torch.zeros_like(embed))
                partial = None
            if use_cache:
                a, kv = layer.attn(layer.attn_norm(h), self.rope_cos, self.rope_sin, mask,
                                   past_kv[i] if past_kv is not None else None, use_cache=True)
                new_kv.append(kv)
            else:
                a = layer.attn(layer.attn_norm(h), self.rope_cos, self.rope_sin, mask)
            partial = a if partial is None else partial + a
            h = route_sources(committed + [partial], layer.mlp_res_query, layer.mlp_res_norm.weight,
                              layer.mlp_res_norm.eps)
            partial = partial + layer.ffn(layer.ffn_norm(h))
            if collect is not None:
                collect.append(h)
        x = route_sources(committed + [partial], self.final_res_query, self.final_res_norm.weight,
                          self.final_res_norm.eps)
        return self.norm(x), new_kv

    # ---- forward --------------------------------------------------------
    def hidden_states(self, input_ids: torch.Tensor, mask: Optional[torch.Tensor] = None, past_kv: Any = None,
                      use_cache: bool = False) -> tuple[torch.Tensor, list]:
        x = self.embed_tokens(input_ids)
        if self.config.attn_res:
            return self._forward_attn_res(x, mask, past_kv, use_cache)
        new_kv: list = []
        for i, layer in enumerate(self.layers):
            if use_cache:
                x, kv = layer(x, self.rope_cos, self.rope_sin, mask,
                              past_kv[i] if past_kv is not None else None, use_cache=True)
                new_kv.append(kv)
            elif self.config.activation_checkpointing and self.training:
                from torch.utils.checkpoint import checkpoint
                x = checkpoint(layer, x, self.rope_cos, self.rope_sin, mask, use_reentrant=False)
            else:
                x = layer(x, self.rope_cos, self.rope_sin, mask)
        return self.norm(x), new_kv

    def loss_from_logits(self, logits: torch.Tensor, labels: torch.Tensor) -> dict[str, torch.Tensor]:
        sl = logits[..., :-1, :].reshape(-1, logits.size(-1))
        sl = sl if sl.dtype == torch.float64 else sl.float()
        tl = labels[..., 1:].reshape(-1)
        out: dict[str, torch.Tensor] = {}
        loss = F.cross_entropy(sl, tl, ignore_index=-100)
        if self.config.z_loss_weight > 0:
            z = self.config.z_loss_weight * (torch.logsumexp(sl, -1) ** 2).mean()
            loss = loss + z
            out["z_loss"] = z
        out["loss"] = loss
        return out

    def forward(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
                mask: Optional[torch.Tensor] = None, past_kv: Any = None, use_cache: bool = False
                ) -> dict[str, Any]:
        x, new_kv = self.hidden_states(input_ids, mask, past_kv, use_cache)
        out: dict[str, Any] = {}
        if use_cache:
            out["past_kv"] = new_kv
        logits = F.linear(x, self.get_lm_head_weight())
        out["logits"] = logits
        if labels is not None:
            out.update(self.loss_from_logits(logits, labels))
        return out


# Names under which the reference exposes the same objects.
LuxiaBaseModel = KotodamaModel
LuxiaModelConfig = ModelConfig
