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
    all_to_all_rows: Optional[Callable] = None
    runtime: Optional["EpRuntime"] = None     # peer-memory data plane (GPUs)


class EpRuntime:
    """Symmetric receive buffers and epochs for the peer-memory dispatch/combine kernels
    (``csrc/moe/ep.cu``).  ``capacity_factor`` bounds the rows one rank may receive relative to
    a perfectly balanced routing; an overflow is detected on the device, identically on every
    rank, and surfaces as an error from ``SymmHeap.check``."""

    def __init__(self, heap, num_experts: int, hidden: int, max_tokens: int, top_k: int,
                 capacity_factor: float = 2.0):
        if num_experts % heap.world:
            raise ValueError(f"{num_experts} experts do not split over {heap.world} ranks")
        self.heap = heap
        self.E, self.E_local, self.H = num_experts, num_experts // heap.world, hidden
        pairs = max_tokens * top_k
        factor = 1.0 if heap.world == 1 else capacity_factor
        self.cap_rows = (int(pairs * factor) + self.E_local * 128 + 127) // 128 * 128
        self.xs = heap.alloc(self.cap_rows * hidden * 2)
        self.ys = heap.alloc(self.cap_rows * hidden * 2)
        self.counts_all = heap.alloc(heap.world * num_experts * 4)
        # barrier flags of the two kernels and their device-resident call number (the kernels advance it themselves, so
        # the decode step can be captured in a CUDA graph and replayed)
        from .symm import MAX_RANKS
        self.flags = heap.alloc((3 * MAX_RANKS + 4) * 4)
        self.flags.local.zero_()
        if torch.device(heap.device).type == "cuda":
            torch.cuda.synchronize(heap.device)
        if heap.world > 1:
            heap.comm.barrier()     # nobody signals into flags that are still being cleared

    def view(self, buf) -> torch.Tensor:
        return buf.local.view(torch.bfloat16)[:self.cap_rows * self.H].view(self.cap_rows, self.H)

    def experts(self, x, scores, idx, counts, gate_up, down, act, gate_up_t=None, down_t=None):
        from ..ops import cuda as C
        return _EpExperts.apply(x, scores, idx, counts, gate_up, down, gate_up_t, down_t, C._ACT[act], self)


class _EpExperts(torch.autograd.Function):
    """Routed experts sharded over ranks: dispatch (push) -> local grouped GEMMs -> combine (pull).
    The backward pass sends the weighted cotangents along the same plan."""

    @staticmethod
    def forward(ctx, x, scores, idx, counts, gate_up, down, gate_up_t, down_t, act, rt):
        from ..ops import cuda as C
        L, h = C.lib(), rt.heap
        h.guard()
        T, k = idx.shape
        dev = x.device
        dest_row = torch.empty(T * k, dtype=torch.int32, device=dev)
        tile_expert = torch.full((rt.cap_rows // 128,), -1, dtype=torch.int32, device=dev)
        local_rows = torch.zeros(1, dtype=torch.int32, device=dev)
        xc = x.contiguous()
        L.ep_dispatch(xc, idx, None, counts, rt.counts_all.ptrs, rt.xs.ptrs, rt.flags.ptrs, h.rank, h.world,
                      0, h.wait_limit_s, rt.cap_rows, dest_row, tile_expert, local_rows, False, h.abort_word)
        need = x.requires_grad or scores.requires_grad
        # unused tiles are never written nor read back; the zero fill is kept where the rows are saved for backward
        o1 = None if need else torch.empty(rt.cap_rows, gate_up.shape[1], dtype=torch.bfloat16, device=dev)
        gu = L.moe_grouped_gemm(rt.view(rt.xs), gate_up, tile_expert, o1)
        hh = L.glu_fwd(gu, act)
        L.moe_grouped_gemm(hh, down, tile_expert, rt.view(rt.ys))
        del hh
        sc = scores.float().contiguous()
        keep = torch.empty(T * k, x.shape[1], dtype=torch.bfloat16, device=dev) if need else None
        out = L.ep_combine(rt.ys.ptrs, idx, dest_row, sc, x.shape[1], rt.E_local, rt.flags.ptrs, h.rank, h.world,
                           0, h.wait_limit_s, keep, h.abort_word)
        ctx.save_for_backward(gu, keep, sc, idx, counts, dest_row, tile_expert, local_rows, gate_up, down, gate_up_t, down_t)
        ctx.act, ctx.rt, ctx.score_dtype = act, rt, scores.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import cuda as C
        L, rt = C.lib(), ctx.rt
        h = rt.heap
        gu, keep, sc, idx, counts, dest_row, tile_expert, local_rows, gate_up, down, gate_up_t, down_t = ctx.saved_tensors
        T, k = idx.shape
        dout = dout.contiguous()
        ident = torch.arange(T * k, dtype=torch.int32, device=dout.device)
        dsc = L.moe_pair_dot(dout, keep, ident, k).to(ctx.score_dtype)
        L.ep_dispatch(dout, idx, sc.view(-1), counts, rt.counts_all.ptrs, rt.xs.ptrs, rt.flags.ptrs, h.rank, h.world,
                      0, h.wait_limit_s, rt.cap_rows, dest_row, tile_expert, local_rows, True, h.abort_word)
        if down_t is None:
            down_t = down.transpose(1, 2).contiguous()
        dh = L.moe_grouped_gemm(rt.view(rt.xs), down_t, tile_expert)
        dgu = L.glu_bwd(gu, dh, ctx.act)
        del dh
        if gate_up_t is None:
            gate_up_t = gate_up.transpose(1, 2).contiguous()
        L.moe_grouped_gemm(dgu, gate_up_t, tile_expert, rt.view(rt.ys))
        dx = L.ep_combine(rt.ys.ptrs, idx, dest_row, None, dout.shape[1], rt.E_local, rt.flags.ptrs, h.rank, h.world,
                          0, h.wait_limit_s, None, h.abort_word)
        return dx, dsc, None, None, None, None, None, None, None, None


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
    if ctx.runtime is not None and x2.is_cuda and x2.dtype == torch.bfloat16 and router_w.dtype == torch.bfloat16:
        from .. import ops
        from ..ops import cuda as C
        logits = ops.lora_linear(x2, router_w, None, None).float()
        scores, idx, counts, _ = C.moe_route(logits, top_k, True)
        out = ctx.runtime.experts(x2, scores.to(x2.dtype), idx, counts, gate_up, down, act)
        if shared is not None:
            out = out + torch.sigmoid(F.linear(x2, shared_gate_w)) * shared(x2)
        return out.reshape(shape)
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
