"""Hot-op entry points.

Each function takes tensors and runs the hand-written sm_100a kernel when its
inputs live on a GPU, or the eager restatement from ``ops.eager`` when they
live on the CPU (the test oracle and the CPU smoke config).  There is no
silent GPU fallback: a CUDA tensor with the native extension missing raises
``ExtensionMissing`` so a GPU run can never quietly use library kernels.
"""
from __future__ import annotations

from . import eager
from .eager import (apply_rope, default_inv_freq, l2norm, llama3_inv_freq, rope_tables,
                    stable_softplus)


class ExtensionMissing(RuntimeError):
    pass


def _cuda():
    from . import cuda as _c
    return _c


_LIBRARY_BASELINE = False


def use_library_kernels(flag: bool) -> None:
    """Benchmark baseline switch: when set, CUDA tensors run on library kernels instead of this
    package's: the eager restatements in ``ops.eager`` (cuBLAS GEMMs, unfused norms, RoPE, GLU,
    log-softmax), PyTorch's fused SDPA for full-sequence attention and flash-attn's KV-cache kernel
    for decode.  Never set implicitly; the product path leaves it off."""
    global _LIBRARY_BASELINE
    _LIBRARY_BASELINE = bool(flag)


def native(*ts) -> bool:
    """True when the hand-written kernels should handle these tensors."""
    return not _LIBRARY_BASELINE and any(t is not None and t.is_cuda for t in ts)


def _on_gpu(*ts) -> bool:
    return native(*ts)


def rmsnorm(x, weight, eps, zero_centered=False):
    if _on_gpu(x):
        return _cuda().rmsnorm(x, weight, eps, zero_centered)
    return eager.rmsnorm(x, weight, eps, zero_centered)


def add_rmsnorm(x, residual, weight, eps, zero_centered=False):
    if _on_gpu(x):
        return _cuda().add_rmsnorm(x, residual, weight, eps, zero_centered)
    return eager.add_rmsnorm(x, residual, weight, eps, zero_centered)


def rmsnorm_gated(x, gate, weight, eps):
    if _on_gpu(x):
        return _cuda().rmsnorm_gated(x, gate, weight, eps)
    return eager.rmsnorm_gated(x, gate, weight, eps)


def qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered=False):
    if _on_gpu(q):
        return _cuda().qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered)
    return eager.qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered)


def _library_attention(q, k, v, scale, causal):
    """Benchmark baseline: PyTorch's fused SDPA (GQA-native flash kernel) on ``[B,S,H,D]`` tensors."""
    import torch.nn.functional as F
    o = F.scaled_dot_product_attention(q.transpose(1, 2), k.transpose(1, 2), v.transpose(1, 2), is_causal=causal,
                                       scale=scale, enable_gqa=True)
    return o.transpose(1, 2).contiguous()


def _library_decode_attention(q, k_cache, v_cache, kv_len, scale):
    """Benchmark baseline: flash-attn's KV-cache decode kernel (``None`` when the package is missing)."""
    try:
        from flash_attn import flash_attn_with_kvcache
    except ImportError:
        return None
    import torch
    return flash_attn_with_kvcache(q[:, None], k_cache, v_cache, cache_seqlens=kv_len.to(torch.int32),
                                   softmax_scale=scale, causal=True)[:, 0]


def attention(q, k, v, *, scale, causal=True, window=0, q_offset=0, softmax_fp32=True, kv_len=None):
    if _LIBRARY_BASELINE and q.is_cuda and not window and not q_offset and kv_len is None and q.dtype != __import__("torch").float32:
        return _library_attention(q, k, v, scale, causal)
    if _on_gpu(q):
        return _cuda().attention(q, k, v, scale=scale, causal=causal, window=window,
                                 q_offset=q_offset, kv_len=kv_len)
    return eager.attention(q, k, v, scale=scale, causal=causal, window=window, q_offset=q_offset,
                           softmax_fp32=softmax_fp32, kv_len=kv_len)


def decode_attention(q, k_cache, v_cache, kv_len, *, scale, window=0):
    if _LIBRARY_BASELINE and q.is_cuda and not window and k_cache.dim() == 4:
        out = _library_decode_attention(q, k_cache, v_cache, kv_len, scale)
        if out is not None:
            return out
    if _on_gpu(q):
        return _cuda().decode_attention(q, k_cache, v_cache, kv_len, scale=scale, window=window)
    return eager.decode_attention(q, k_cache, v_cache, kv_len, scale=scale, window=window)


def swiglu(gate_up, act="silu"):
    if _on_gpu(gate_up):
        return _cuda().swiglu(gate_up, act)
    return eager.swiglu(gate_up, act)


def lora_linear(x, w, a_stack, b_stack, wt=None, bias=None, residual=None):
    """``y = x Wᵀ + (x Aᵀ) Bᵀ (+ residual)``.  ``wt`` is the optional resident transpose of a
    frozen ``w`` used by the backward GEMM so both passes read K-major tiles."""
    if _on_gpu(x):
        return _cuda().lora_linear(x, w, a_stack, b_stack, wt, bias, residual)
    y = eager.lora_linear(x, w, a_stack, b_stack, bias)
    return y if residual is None else residual + y


def lora_merge(w, a_stack, b_stack):
    if _on_gpu(w):
        return _cuda().lora_merge(w, a_stack, b_stack)
    return eager.lora_merge(w, a_stack, b_stack)


def logprob_gather(hidden, head_w, targets, temperature=1.0, softcap=0.0, head_wt=None):
    if _on_gpu(hidden):
        return _cuda().logprob_gather(hidden, head_w, targets, temperature, softcap, head_wt)
    return eager.logprob_gather(hidden, head_w, targets, temperature, softcap)


def embedding(ids, table, scale=1.0):
    if _on_gpu(table):
        return _cuda().embedding(ids, table, scale)
    return eager.embedding(ids, table, scale)


def sample_top_p(logits, base_seed, global_rows, draw, temperature, top_p, draw_dev=None):
    """``draw_dev`` (int32 device scalar) overrides ``draw`` so a captured CUDA graph can advance it."""
    return _cuda().sample_top_p(logits, base_seed, global_rows, draw, temperature, top_p, draw_dev)


def grpo_loss_fused(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w=None):
    return _cuda().grpo_loss(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w)


def adamw_step(params, grads, m, v, **kw):
    if params and native(params[0]):
        return _cuda().adamw_step(params, grads, m, v, **kw)
    return eager.adamw_step(params, grads, m, v, **kw)
