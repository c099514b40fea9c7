"""Qwen3 binding of the dense backbone: per-head QK RMSNorm before RoPE,
attention in the model dtype, explicit ``head_dim``; ``attention_bias`` and an
active ``sliding_window`` are rejected (reference ``crates/ferrl/src/qwen.rs:35-124``)."""
from __future__ import annotations

from typing import Any, Mapping

from .dense import DenseSpec


def qwen3_spec(cfg: Mapping[str, Any]) -> DenseSpec:
    if cfg.get("attention_bias"):
        raise ValueError("Qwen3 with attention_bias=true is not supported")
    if cfg.get("use_sliding_window") and cfg.get("sliding_window"):
        raise ValueError("Qwen3 with an active sliding_window is not supported")
    rope = cfg.get("rope_parameters") or {}
    theta = float(rope.get("rope_theta", cfg.get("rope_theta", 1e6)))
    if rope.get("rope_type", "default") not in ("default", None):
        raise ValueError(f"unsupported Qwen3 rope_type {rope.get('rope_type')!r}")
    heads = int(cfg["num_attention_heads"])
    spec = DenseSpec(
        vocab_size=int(cfg["vocab_size"]), hidden_size=int(cfg["hidden_size"]),
        num_hidden_layers=int(cfg["num_hidden_layers"]), num_attention_heads=heads,
        num_key_value_heads=int(cfg.get("num_key_value_heads", heads)),
        head_dim=int(cfg.get("head_dim") or int(cfg["hidden_size"]) // heads),
        intermediate_size=int(cfg["intermediate_size"]), rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-6)),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)), qk_norm=True, sdpa_f32=False,
        activation=str(cfg.get("hidden_act", "silu")), rope_theta=theta,
        max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)), family="qwen3")
    spec.validate()
    return spec


def qwen3_8b_spec(max_position_embeddings: int = 4096) -> DenseSpec:
    """The Qwen3-8B geometry used by the headline benchmark."""
    return DenseSpec(vocab_size=151936, hidden_size=4096, num_hidden_layers=36, num_attention_heads=32,
                     num_key_value_heads=8, head_dim=128, intermediate_size=12288, rms_norm_eps=1e-6,
                     tie_word_embeddings=False, qk_norm=True, rope_theta=1e6,
                     max_position_embeddings=max_position_embeddings, family="qwen3")
