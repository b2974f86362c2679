"""Evaluation and analysis helpers (see :mod:`kotodama_b200.eval.core`)."""
from .core import (CheckpointInfo, ForwardResult, compute_attention_weights, compute_perplexity, extract_keys_matching,
                   extract_series, forward_with_states, generate, generate_text, get_nearest_step, get_value,
                   load_checkpoint_registry, load_metrics, load_model, load_model_config, load_multiple)
from . import plot_utils, run_analysis

__all__ = ["load_model", "load_model_config", "load_checkpoint_registry", "CheckpointInfo", "forward_with_states",
           "compute_attention_weights", "ForwardResult", "generate", "generate_text", "compute_perplexity",
           "load_metrics", "get_nearest_step", "get_value", "extract_series", "extract_keys_matching", "load_multiple",
           "run_analysis", "plot_utils"]
