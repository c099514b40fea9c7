"""Plain PyTorch restatements of every hot op.

These run the CPU path (tests, the tiny smoke config) and are the numerical
oracle that each sm_100a kernel in ``csrc/`` is checked against.  Everything
accumulates in float32 and is written the obvious way on purpose.
"""
from __future__ import annotations

import math
from typing import Optional

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------- norms ----
def rmsnorm(x: torch.Tensor, weight: Optional[torch.Tensor], eps: float, zero_centered: bool = False):
    """``x * rsqrt(mean(x^2)+eps) * w`` computed in fp32 then cast back; with
    ``zero_centered`` the scale is ``1 + w`` (reference nn.rs:37-157)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps)
    if weight is not None:
        w = weight.float()
        y = y * ((1.0 + w) if zero_centered else w)
    return y.to(x.dtype)


def rmsnorm_gated(x, gate, weight, eps):
    """``rmsnorm(x) * w * silu(gate)`` (reference nn.rs:169-222)."""
    xf = x.float()
    y = xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * weight.float()
    return (y * F.silu(gate.float())).to(x.dtype)


def add_rmsnorm(x, residual, weight, eps, zero_centered=False):
    """Residual add fused with the following norm: returns ``(norm(h), h)`` with
    ``h = x + residual``."""
    h = x + residual
    return rmsnorm(h, weight, eps, zero_centered), h


def l2norm(x, eps: float = 1e-6):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).sum(-1, keepdim=True) + eps)).to(x.dtype)


def stable_softplus(x):
    return F.softplus(x)


# ----------------------------------------------------------------- rope ----
def rope_tables(inv_freq: torch.Tensor, max_pos: int, device=None):
    t = torch.arange(max_pos, dtype=torch.float32, device=inv_freq.device)
    fr = torch.outer(t, inv_freq.float())
    return fr.cos().to(device), fr.sin().to(device)


def default_inv_freq(rot_dim: int, theta: float) -> torch.Tensor:
    i = torch.arange(0, rot_dim, 2, dtype=torch.float64)
    return (1.0 / (theta ** (i / rot_dim))).float()


def llama3_inv_freq(rot_dim, theta, factor, low_freq_factor, high_freq_factor, original_max_pos):
    """Llama-3 wavelength smoothing (reference llama.rs:59-88)."""
    base = default_inv_freq(rot_dim, theta)
    low_w = original_max_pos / low_freq_factor
    high_w = original_max_pos / high_freq_factor
    out = []
    for f in base.tolist():
        w = 2.0 * math.pi / f
        if w < high_w:
            out.append(f)
        elif w > low_w:
            out.append(f / factor)
        else:
            s = (original_max_pos / w - low_freq_factor) / (high_freq_factor - low_freq_factor)
            out.append((1.0 - s) * f / factor + s * f)
    return torch.tensor(out, dtype=torch.float32)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor):
    """Rotate-half RoPE on the leading ``2*cos.shape[-1]`` channels of the last
    dim. ``x`` ``[B, S, H, D]``; ``positions`` ``[B, S]`` or ``[S]`` (int64);
    tables ``[max_pos, rot/2]``.  Channels past the rotary width pass through
    (partial RoPE, reference blocks.rs:225-244)."""
    half = cos.shape[-1]
    rot = 2 * half
    if positions.dim() == 1:
        positions = positions[None, :].expand(x.shape[0], -1)
    c = cos[positions].unsqueeze(2).float()  # [B,S,1,half]
    s = sin[positions].unsqueeze(2).float()
    xr = x[..., :rot].float()
    x1, x2 = xr[..., :half], xr[..., half:]
    out = torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)
    if rot == x.shape[-1]:
        return out
    return torch.cat([out, x[..., rot:]], dim=-1)


def qk_norm_rope(q, k, q_w, k_w, eps, cos, sin, positions, zero_centered=False):
    """Per-head RMSNorm of q and k (skipped when the weights are ``None``)
    followed by RoPE. ``q`` ``[B,S,Hq,D]``, ``k`` ``[B,S,Hkv,D]``."""
    if q_w is not None:
        q = rmsnorm(q, q_w, eps, zero_centered)
        k = rmsnorm(k, k_w, eps, zero_centered)
    return apply_rope(q, cos, sin, positions), apply_rope(k, cos, sin, positions)


# ------------------------------------------------------------ attention ----
def attention(q, k, v, *, scale: float, causal: bool = True, window: int = 0,
              q_offset: int = 0, softmax_fp32: bool = True, kv_len: Optional[torch.Tensor] = None):
    """GQA attention. ``q`` ``[B,Sq,Hq,D]``, ``k``/``v`` ``[B,Sk,Hkv,D]``.
    Query ``i`` sits at absolute position ``q_offset + i`` and sees keys
    ``j <= pos`` (causal) and ``j > pos - window`` (sliding window, ``window>0``).
    ``kv_len`` ``[B]`` masks keys at or beyond each row's cache length."""
    B, Sq, Hq, D = q.shape
    Sk, Hkv = k.shape[1], k.shape[2]
    rep = Hq // Hkv
    qf = q.permute(0, 2, 1, 3)
    kf = k.permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    vf = v.permute(0, 2, 1, 3).repeat_interleave(rep, dim=1)
    if softmax_fp32:
        qf, kf, vf = qf.float(), kf.float(), vf.float()
    scores = torch.matmul(qf, kf.transpose(-1, -2)) * scale
    qi = torch.arange(Sq, device=q.device)[:, None] + q_offset
    kj = torch.arange(Sk, device=q.device)[None, :]
    allowed = torch.ones(Sq, Sk, dtype=torch.bool, device=q.device)
    if causal:
        allowed &= kj <= qi
    if window and window > 0:
        allowed &= kj > qi - window
    allowed = allowed[None, None]
    if kv_len is not None:
        allowed = allowed & (kj[None, None] < kv_len.view(B, 1, 1, 1))
    scores = scores.masked_fill(~allowed, float("-inf"))
    p = torch.softmax(scores.float(), dim=-1).to(vf.dtype)
    p = torch.nan_to_num(p)  # rows with no visible key
    out = torch.matmul(p, vf)
    return out.permute(0, 2, 1, 3).to(q.dtype).contiguous()


def decode_attention(q, k_cache, v_cache, kv_len, *, scale: float, window: int = 0):
    """One new token per row against a dense cache. ``q`` ``[B,Hq,D]``, caches
    ``[B,Smax,Hkv,D]``, ``kv_len`` ``[B]`` counts valid keys *including* the new
    token (already written)."""
    B, Hq, D = q.shape
    Smax = k_cache.shape[1]
    kj = torch.arange(Smax, device=q.device)[None, :]
    allowed = kj < kv_len[:, None]
    if window and window > 0:
        allowed &= kj >= (kv_len[:, None] - window)
    Hkv = k_cache.shape[2]
    rep = Hq // Hkv
    kf = k_cache.float().repeat_interleave(rep, dim=2)  # [B,S,Hq,D]
    vf = v_cache.float().repeat_interleave(rep, dim=2)
    scores = torch.einsum("bhd,bshd->bhs", q.float(), kf) * scale
    scores = scores.masked_fill(~allowed[:, None, :], float("-inf"))
    p = torch.softmax(scores, dim=-1)
    p = torch.where(allowed.any(dim=1)[:, None, None], p, torch.zeros_like(p))   # a row with no keys attends to nothing
    return torch.einsum("bhs,bshd->bhd", p, vf).to(q.dtype)


# ------------------------------------------------------------ mlp / act ----
def swiglu(gate_up: torch.Tensor, act: str = "silu"):
    """``act(gate) * up`` on a fused ``[..., 2F]`` tensor laid out ``[gate | up]``."""
    g, u = gate_up.chunk(2, dim=-1)
    if act == "silu":
        a = F.silu(g.float())
    elif act in ("gelu_pytorch_tanh", "gelu_tanh"):
        a = F.gelu(g.float(), approximate="tanh")
    elif act == "gelu":
        a = F.gelu(g.float())
    else:
        raise ValueError(f"unsupported activation {act}")
    return (a * u.float()).to(gate_up.dtype)


# ----------------------------------------------------------------- lora ----
def lora_linear(x, w, a_stack, b_stack, bias=None):
    """``y = x Wᵀ + (x Aᵀ) Bᵀ``; ``a_stack`` ``[R, in]``, ``b_stack`` ``[out, R]``
    already carry the LoRA scale (in ``b_stack``). Either may be ``None``."""
    y = F.linear(x, w, bias)
    if a_stack is not None:
        t = F.linear(x, a_stack.to(x.dtype))
        y = y + F.linear(t, b_stack.to(x.dtype))
    return y


def lora_merge(w, a_stack, b_stack):
    """``W + B A`` in fp32, cast to ``w.dtype`` (reference lora.rs:1335-1350)."""
    if a_stack is None:
        return w
    return (w.float() + b_stack.float() @ a_stack.float()).to(w.dtype)


# -------------------------------------------------------------- logprob ----
def logprob_gather(hidden, head_w, targets, temperature: float = 1.0, softcap: float = 0.0,
                   chunk: int = 128):
    """Per-token ``log_softmax(h Wᵀ / T)[target]`` without keeping ``[N, V]``
    beyond one chunk of rows (reference model.rs:523-559). ``hidden`` ``[N, H]``,
    ``targets`` ``[N]`` -> ``[N]`` float32.  ``softcap>0`` applies
    ``cap*tanh(x/cap)`` to the logits first (Gemma)."""
    outs = []
    for s in range(0, hidden.shape[0], chunk):
        h = hidden[s:s + chunk]
        logits = F.linear(h, head_w).float()
        if softcap and softcap > 0:
            logits = softcap * torch.tanh(logits / softcap)
        logits = logits / temperature
        lp = torch.log_softmax(logits, dim=-1)
        outs.append(lp.gather(-1, targets[s:s + chunk, None].long()).squeeze(-1))
    return torch.cat(outs) if outs else hidden.new_zeros(0, dtype=torch.float32)


def embedding(ids, table, scale: float = 1.0):
    e = F.embedding(ids, table)
    return e if scale == 1.0 else (e.float() * scale).to(e.dtype)


# ---------------------------------------------------------------- adamw ----
def adamw_step(params, grads, m, v, *, lr, beta1, beta2, eps, weight_decay, step, grad_scale=1.0):
    """Decoupled AdamW, epsilon outside the square root, bias correction by
    step count (reference optim.rs:257-296).  In place on lists of fp32 tensors."""
    bc1 = 1.0 - beta1 ** step
    bc2 = 1.0 - beta2 ** step
    for p, g, mi, vi in zip(params, grads, m, v):
        g = g * grad_scale if grad_scale != 1.0 else g
        if weight_decay != 0.0:
            p.mul_(1.0 - lr * weight_decay)
        mi.mul_(beta1).add_(g, alpha=1.0 - beta1)
        vi.mul_(beta2).addcmul_(g, g, value=1.0 - beta2)
        denom = (vi / bc2).sqrt_().add_(eps)
        p.addcdiv_(mi / bc1, denom, value=-lr)
