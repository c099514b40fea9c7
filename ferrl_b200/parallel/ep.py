"""Expert parallelism for sparse-MoE layers.

The reference replicates every expert on every rank and walks them in a host
loop (``crates/ferrl/src/moe.rs:122-157``); expert parallelism is a capability
added here.  With an ``EpContext`` installed, experts are sharded over ranks:
tokens are routed on the device, sorted by destination expert, exchanged with
an all-to-all (dispatch), run through the local experts' grouped SwiGLU GEMM,
exchanged back (combine) and weighted into their source rows.  Without a
context (single GPU, CPU tests) the same routing plan runs locally.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable, Optional

import torch
import torch.nn.functional as F

from ..models import moe as M

_CTX: Optional["EpContext"] = None


@dataclass
class EpContext:
    """Expert-parallel group: ``rank`` of ``world`` owns experts ``[rank*E/world, (rank+1)*E/world)``.
    ``all_to_all(send [world, ...rows], send_counts) -> (recv, recv_counts)`` is provided by the
    communicator layer (NCCL baseline or the peer-memory kernel)."""

    rank: int
    world: int
    all_to_all_rows: Callable


def install(ctx: Optional[EpContext]) -> None:
    global _CTX
    _CTX = ctx


def current() -> Optional[EpContext]:
    return _CTX


def sparse_moe(x, router_w, gate_up, down, top_k: int, shared, shared_gate_w, act: str = "silu"):
    """MoE block entry used by the models. ``gate_up``/``down`` hold the LOCAL experts
    (all of them when no expert-parallel context is installed)."""
    ctx = _CTX
    if ctx is None or ctx.world == 1:
        return M.sparse_moe_block(x, router_w, gate_up, down, top_k, shared, shared_gate_w, act)
    shape = x.shape
    x2 = x.reshape(-1, shape[-1])
    E_local = gate_up.shape[0]
    E = E_local * ctx.world
    _, scores, idx = M.topk_router(x2, router_w, top_k)
    plan = M.DispatchPlan.build(idx, E)
    xs = x2[plan.token]                                   # rows sorted by global expert => by destination rank
    per_rank = plan.counts.view(ctx.world, E_local).sum(1)
    recv, recv_counts, recv_expert_counts = ctx.all_to_all_rows(xs, per_rank, plan.counts.view(ctx.world, E_local))
    # received rows arrive grouped by source rank, each group sorted by local expert: regroup by expert
    src_rank_of_row = torch.repeat_interleave(torch.arange(ctx.world, device=x.device), recv_counts)
    local_e = torch.cat([torch.repeat_interleave(torch.arange(E_local, device=x.device), recv_expert_counts[r])
                         for r in range(ctx.world)]) if recv.shape[0] else torch.zeros(0, dtype=torch.long, device=x.device)
    order = torch.sort(local_e, stable=True).indices
    offsets = torch.zeros(E_local + 1, dtype=torch.long, device=x.device)
    offsets[1:] = torch.bincount(local_e, minlength=E_local).cumsum(0)
    ys_sorted = M.grouped_swiglu(recv[order], offsets, gate_up, down, act)
    ys = torch.empty_like(ys_sorted)
    ys[order] = ys_sorted
    back, _, _ = ctx.all_to_all_rows(ys, recv_counts, None)   # combine: return rows to their owners
    del src_rank_of_row
    w = scores.reshape(-1)[plan.order].to(back.dtype).unsqueeze(-1)
    out = torch.zeros_like(x2)
    out.index_add_(0, plan.token, back * w)
    if shared is not None:
        out = out + torch.sigmoid(F.linear(x2, shared_gate_w)) * shared(x2)
    return out.reshape(shape)
