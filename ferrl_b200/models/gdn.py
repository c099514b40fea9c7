"""GatedDeltaNet primitives (Qwen3.5/3.6 linear-attention layers).

Reference: ``crates/ferrl/src/gdn.rs`` - ``stable_softplus`` ``:52``, ``l2norm``
(eps inside the rsqrt of the sum of squares) ``:70``, causal depthwise conv
with a left-context state ``:102-142``, the single-step recurrent delta rule
``:286-317`` and the chunked WY form with carried state ``:451-556`` (chunk 64).

State per head is ``S [k, v]`` (float32).  One token does::

    S <- S * exp(g_t);  delta = (v_t - S^T k_t) * beta_t;  S <- S + k_t delta^T;  o_t = S^T (q_t / sqrt(k))

The chunked form processes C tokens at once.  With cumulative log-decay
``G_i`` inside the chunk, ``L = tril(k_beta k^T * exp(G_i - G_j), -1)`` and
``T = (I + L)^{-1}`` (a unit lower-triangular solve rather than the reference's
8x8 block forward substitution): ``u = T v_beta``, ``w = T (k_beta * exp(G))``,
``v_new = u - w S``, ``o = (q * exp(G)) S + tril(q k^T * decay) v_new`` and
``S <- S exp(G_C) + (k * exp(G_C - G))^T v_new``.

Everything here is differentiable PyTorch and doubles as the oracle for the
sm_100a kernels in ``csrc/kernels/gdn.cu`` (decode step and causal conv), which
``ferrl_b200.ops`` dispatches to on GPUs.
"""
from __future__ import annotations

from typing import Optional

import torch
import torch.nn.functional as F

GDN_CHUNK_SIZE = 64


def stable_softplus(x: torch.Tensor) -> torch.Tensor:
    return F.softplus(x)


def l2norm(x: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    return x * torch.rsqrt((x * x).sum(-1, keepdim=True) + eps)


def causal_depthwise_conv1d(x: torch.Tensor, weight: torch.Tensor, left: Optional[torch.Tensor] = None,
                            activation: bool = False):
    """``x`` ``[B, C, L]``, ``weight`` ``[C, K]``; output ``y[t] = sum_j w[j] x[t-K+1+j]``
    with ``left`` ``[B, C, K-1]`` (zeros if absent) as the context before ``t=0``.
    Returns ``(y, new_left)`` where ``new_left`` is the last ``K-1`` inputs."""
    B, C, L = x.shape
    K = weight.shape[-1]
    if left is None:
        left = x.new_zeros(B, C, K - 1)
    xx = torch.cat([left.to(x.dtype), x], dim=-1)
    y = F.conv1d(xx, weight.to(x.dtype).unsqueeze(1), None, padding=0, groups=C)
    if activation:
        y = F.silu(y)
    return y, xx[:, :, -(K - 1):] if K > 1 else xx[:, :, :0]


def gated_delta_rule_recurrent(q, k, v, g, beta, state: Optional[torch.Tensor] = None, use_qk_l2norm: bool = False):
    """Token-by-token form. ``q,k`` ``[B,T,H,K]``, ``v`` ``[B,T,H,V]``, ``g,beta`` ``[B,T,H]``;
    ``state`` ``[B,H,K,V]``. Returns ``(out [B,T,H,V], state)`` in float32 math."""
    dt = q.dtype
    if use_qk_l2norm:
        q, k = l2norm(q.float()), l2norm(k.float())
    q, k, v, g, beta = (t.float().transpose(1, 2) for t in (q, k, v, g, beta))
    B, H, T, Kd = k.shape
    Vd = v.shape[-1]
    q = q * (Kd ** -0.5)
    S = q.new_zeros(B, H, Kd, Vd) if state is None else state.float()
    outs = []
    for t in range(T):
        S = S * g[:, :, t].exp()[..., None, None]
        kv = (S * k[:, :, t].unsqueeze(-1)).sum(-2)
        delta = (v[:, :, t] - kv) * beta[:, :, t].unsqueeze(-1)
        S = S + k[:, :, t].unsqueeze(-1) * delta.unsqueeze(-2)
        outs.append((S * q[:, :, t].unsqueeze(-1)).sum(-2))
    out = torch.stack(outs, dim=2).transpose(1, 2).contiguous().to(dt)
    return out, S


def gated_delta_rule_chunked(q, k, v, g, beta, state: Optional[torch.Tensor] = None, chunk: int = GDN_CHUNK_SIZE,
                             use_qk_l2norm: bool = False):
    """Chunked (WY) form, numerically equal to the recurrent form."""
    dt = q.dtype
    if use_qk_l2norm:
        q, k = l2norm(q.float()), l2norm(k.float())
    q, k, v, g, beta = (t.float().transpose(1, 2).contiguous() for t in (q, k, v, g, beta))
    B, H, T, Kd = k.shape
    Vd = v.shape[-1]
    pad = (chunk - T % chunk) % chunk
    if pad:
        q, k, v = (F.pad(t, (0, 0, 0, pad)) for t in (q, k, v))
        g, beta = F.pad(g, (0, pad)), F.pad(beta, (0, pad))
    n = (T + pad) // chunk
    q = q * (Kd ** -0.5)
    kb, vb = k * beta.unsqueeze(-1), v * beta.unsqueeze(-1)
    shp = lambda t: t.reshape(B, H, n, chunk, t.shape[-1])  # noqa: E731
    q, k, kb, vb = shp(q), shp(k), shp(kb), shp(vb)
    G = g.reshape(B, H, n, chunk).cumsum(-1)
    diff = G.unsqueeze(-1) - G.unsqueeze(-2)                      # G_i - G_j
    tril = torch.ones(chunk, chunk, dtype=torch.bool, device=q.device).tril()
    decay = torch.where(tril, diff, torch.zeros_like(diff)).exp() * tril   # exp only where i >= j (no overflow)
    L = (kb @ k.transpose(-1, -2)) * decay
    L = L * torch.ones(chunk, chunk, device=q.device).tril(-1)
    eye = torch.eye(chunk, device=q.device, dtype=q.dtype)
    Tm = torch.linalg.solve_triangular(eye + L, eye.expand_as(L).contiguous(), upper=False)
    u = Tm @ vb
    w = Tm @ (kb * G.exp().unsqueeze(-1))
    S = q.new_zeros(B, H, Kd, Vd) if state is None else state.float()
    outs = []
    for i in range(n):
        qi, ki = q[:, :, i], k[:, :, i]
        attn = (qi @ ki.transpose(-1, -2)) * decay[:, :, i]
        v_new = u[:, :, i] - w[:, :, i] @ S
        o = (qi * G[:, :, i].exp().unsqueeze(-1)) @ S + attn @ v_new
        outs.append(o)
        last = G[:, :, i, -1]
        S = S * last.exp()[..., None, None] + (ki * (last.unsqueeze(-1) - G[:, :, i]).exp().unsqueeze(-1)).transpose(-1, -2) @ v_new
    out = torch.cat(outs, dim=2)[:, :, :T].transpose(1, 2).contiguous().to(dt)
    return out, S
