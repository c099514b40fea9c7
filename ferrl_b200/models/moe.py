"""Sparse mixture-of-experts primitives.

Reference (``crates/ferrl/src/moe.rs``): ``topk_router`` - float32 softmax over
experts, top-k, renormalise ``:74-89``; ``moe_experts`` - a host loop over
experts with a device->host copy of the routing table per layer, gather /
SwiGLU / ``index_add`` ``:110-158``; ``sparse_moe_block`` adds a sigmoid-gated
shared expert ``:172-190``.

Here routing never leaves the device.  Token->expert assignments are sorted by
expert (one stable sort of ``T*k`` keys), giving a permutation and per-expert
segment offsets; the experts then run as a *grouped* SwiGLU GEMM over ragged
segments and the weighted results are scattered back.  Empty experts are just
empty segments.  On CPU (and as the oracle for the kernels) the grouped GEMM is
a loop over non-empty segments of the sorted buffer; on GPUs
``ferrl_b200.parallel.ep`` runs the same plan with the permute fused into the
expert-parallel all-to-all dispatch and the tcgen05 grouped GEMM.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.nn.functional as F


def ops_native(t):
    from .. import ops
    return ops.native(t)


def topk_router(x: torch.Tensor, weight: torch.Tensor, top_k: int, renorm: bool = True):
    """``x`` ``[T, H]``, router ``weight`` ``[E, H]`` -> ``(probs [T,E] f32, scores [T,k] f32, indices [T,k])``."""
    logits = F.linear(x, weight)
    probs = torch.softmax(logits.float(), dim=-1)
    scores, idx = torch.topk(probs, top_k, dim=-1)
    if renorm:
        scores = scores / scores.sum(-1, keepdim=True)
    return probs, scores, idx


@dataclass
class DispatchPlan:
    """Sorted-by-expert view of the ``T*k`` (token, slot) assignments."""

    order: torch.Tensor       # [T*k] positions into the flattened (token, slot) list, sorted by expert
    token: torch.Tensor       # [T*k] source token of each sorted row
    counts: torch.Tensor      # [E] rows per expert
    offsets: torch.Tensor     # [E+1] segment starts

    @staticmethod
    def build(indices: torch.Tensor, num_experts: int) -> "DispatchPlan":
        T, k = indices.shape
        flat = indices.reshape(-1)
        order = torch.sort(flat, stable=True).indices
        counts = torch.bincount(flat, minlength=num_experts)
        offsets = torch.zeros(num_experts + 1, dtype=torch.long, device=indices.device)
        offsets[1:] = counts.cumsum(0)
        return DispatchPlan(order, order // k, counts, offsets)


def grouped_swiglu(xs: torch.Tensor, offsets: torch.Tensor, gate_up: torch.Tensor, down: torch.Tensor,
                   act: str = "silu") -> torch.Tensor:
    """Ragged grouped expert MLP over rows already sorted by expert.
    ``gate_up`` ``[E, 2I, H]`` (rows ``[gate | up]``), ``down`` ``[E, H, I]``."""
    out = torch.zeros_like(xs)
    offs = offsets.tolist()
    for e in range(gate_up.shape[0]):
        a, b = offs[e], offs[e + 1]
        if a == b:
            continue
        g, u = F.linear(xs[a:b], gate_up[e]).chunk(2, dim=-1)
        h = (F.silu(g) if act == "silu" else F.gelu(g, approximate="tanh")) * u
        out[a:b] = F.linear(h, down[e])
    return out


def moe_experts(x: torch.Tensor, indices: torch.Tensor, scores: torch.Tensor, gate_up: torch.Tensor,
                down: torch.Tensor, act: str = "silu") -> torch.Tensor:
    """Routed experts: permute -> grouped SwiGLU -> weight -> scatter-add. ``x`` ``[T,H]``."""
    E = gate_up.shape[0]
    plan = DispatchPlan.build(indices, E)
    xs = x[plan.token]
    ys = grouped_swiglu(xs, plan.offsets, gate_up, down, act)
    w = scores.reshape(-1)[plan.order].to(ys.dtype).unsqueeze(-1)
    out = torch.zeros_like(x)
    out.index_add_(0, plan.token, ys * w)
    return out


def _device_moe(x2, router_w, gate_up, down, top_k, act, gate_up_t=None, down_t=None):
    """Device-resident plan: router kernel, counting-sort dispatch into 128-row expert segments,
    tcgen05 grouped GEMMs, deterministic combine (``csrc/moe/moe.cu``).  ``None`` when the
    tensors are outside the kernels' domain."""
    if x2.dtype != torch.bfloat16 or router_w.dtype != torch.bfloat16 or router_w.shape[0] > 1024 or top_k > 16:
        return None
    from .. import ops
    from ..ops import cuda as C
    logits = ops.lora_linear(x2, router_w, None, None).float()
    scores, idx, counts, _ = C.moe_route(logits, top_k, True)
    # the eager plan rounds the routing weights to the activation dtype before use
    return C.moe_experts(x2, scores.to(x2.dtype), idx, counts, gate_up, down, act, gate_up_t, down_t)


def sparse_moe_block(x: torch.Tensor, router_w, gate_up, down, top_k: int, shared=None, shared_gate_w=None,
                     act: str = "silu") -> torch.Tensor:
    """``x`` ``[..., H]``. ``shared`` is a callable shared-expert MLP, gated by
    ``sigmoid(x @ shared_gate_w^T)``."""
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    y = _device_moe(x2, router_w, gate_up, down, top_k, act) if ops_native(x2) else None
    if y is None:
        _, scores, idx = topk_router(x2, router_w, top_k)
        y = moe_experts(x2, idx, scores.to(x2.dtype), gate_up, down, act)
    if shared is not None:
        y = y + torch.sigmoid(F.linear(x2, shared_gate_w)) * shared(x2)
    return y.reshape(shape)
