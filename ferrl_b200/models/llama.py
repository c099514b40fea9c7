"""Llama-3.x binding of the dense backbone: no QK-norm, fp32 softmax, derived
``head_dim = hidden / heads``, optional llama3 RoPE wavelength smoothing
(reference ``crates/ferrl/src/llama.rs:59-190``).  Library API only: the CLI
auto-loader never selects it, as in the reference."""
from __future__ import annotations

from typing import Any, Mapping

from .. import ops
from .dense import DenseSpec


def llama_spec(cfg: Mapping[str, Any]) -> DenseSpec:
    heads = int(cfg["num_attention_heads"])
    hidden = int(cfg["hidden_size"])
    head_dim = int(cfg.get("head_dim") or hidden // heads)
    rope = cfg.get("rope_parameters") or {}
    theta = float(rope.get("rope_theta", cfg.get("rope_theta", 10000.0)))
    scaling = cfg.get("rope_scaling") or (rope if rope.get("rope_type") not in (None, "default") else None)
    inv = None
    if scaling and scaling.get("rope_type", scaling.get("type", "default")) == "llama3":
        inv = ops.llama3_inv_freq(head_dim, theta, float(scaling["factor"]), float(scaling["low_freq_factor"]),
                                  float(scaling["high_freq_factor"]),
                                  float(scaling["original_max_position_embeddings"]))
    elif scaling and scaling.get("rope_type", scaling.get("type", "default")) not in ("default", None):
        raise ValueError(f"unsupported llama rope scaling {scaling!r}")
    if cfg.get("attention_bias") or cfg.get("mlp_bias"):
        raise ValueError("Llama with projection biases is not supported")
    spec = DenseSpec(
        vocab_size=int(cfg["vocab_size"]), hidden_size=hidden, num_hidden_layers=int(cfg["num_hidden_layers"]),
        num_attention_heads=heads, num_key_value_heads=int(cfg.get("num_key_value_heads", heads)),
        head_dim=head_dim, intermediate_size=int(cfg["intermediate_size"]),
        rms_norm_eps=float(cfg.get("rms_norm_eps", 1e-5)),
        tie_word_embeddings=bool(cfg.get("tie_word_embeddings", False)), qk_norm=False, sdpa_f32=True,
        activation="silu", rope_theta=theta, max_position_embeddings=int(cfg.get("max_position_embeddings", 4096)),
        inv_freq=inv, family="llama")
    spec.validate()
    return spec
