"""Sequence-sharded tensor parallelism: the residual stream holds 1 / world of the token rows.

Between a row-parallel projection and the next column-parallel one the plain Megatron layout keeps the
``[tokens, hidden]`` activation replicated: the row-parallel output is all-reduced and every rank runs the
norms and the residual add on all rows.  Here the row-parallel partial is reduce-scattered over the token rows
instead (each rank sums and keeps ``tokens / world`` rows), norms and residual run on that shard, and the next
column-parallel projection all-gathers the normalised rows.  The two collectives move the same bytes as the one
all-reduce they replace, the elementwise work and the activations kept for the backward pass shrink by ``world``.

Four differentiable row collectives on ``[rows, hidden]`` tensors (rows a multiple of the world size, shards are
contiguous row blocks):

``gather_rows_tp``        all-gather whose consumer is rank-specific (a column-parallel projection): the backward
                           is a reduce-scatter of the ranks' different gradients.
``gather_rows_replicated`` all-gather whose consumer is computed identically on every rank (final norm, head, loss):
                           the backward takes this rank's rows of the (identical) gradient.
``scatter_rows_sum``      reduce-scatter of row-parallel partials: the backward is an all-gather.
``shard_rows``            this rank's rows of a replicated tensor: the backward all-gathers (embedding output).

On GPUs with a registered ``RowCollectives`` they run as cooperative kernels over the symmetric heap
(``csrc/dp/dp_step.cu``: ``symm_reduce_scatter_kernel`` / ``symm_all_gather_kernel``, bounded barriers, rank-ordered
sums); otherwise through the ``Comm`` seam.  The reference has no sequence sharding: it all-reduces the
``[b, l, hidden]`` partial after every row-parallel projection (``crates/ferrl/src/tensor_parallel.rs:417-462``).
"""
from __future__ import annotations

from typing import Optional

import torch

from ..comm import Comm
from .symm import SymmHeap

_ROW_COLLECTIVES: dict = {}


class RowCollectives:
    """Staging buffer and launches of the two row-collective kernels for one communicator."""

    def __init__(self, heap: SymmHeap, max_bytes: int):
        self.heap = heap
        self.buf = heap.alloc(max_bytes)
        self.max_bytes = max_bytes

    def _ok(self, x, nbytes):
        return x.is_cuda and x.dtype in (torch.bfloat16, torch.float32) and 0 < nbytes <= self.max_bytes

    def reduce_scatter(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        h = self.heap
        rows = x.shape[0]
        nbytes = x.numel() * x.element_size()
        if rows % h.world or not self._ok(x, nbytes):
            return None
        h.guard()
        self.buf.local[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        out = torch.empty((rows // h.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        h.C.lib().symm_row_collective(0, self.buf.ptrs, h.flags.ptrs, out, out.numel(), h.rank, h.world, h.next_epoch(),
                                      h.wait_limit_s, h.abort_word)
        return out

    def all_gather(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        h = self.heap
        nbytes = x.numel() * x.element_size()
        if not self._ok(x, nbytes * h.world):
            return None
        h.guard()
        self.buf.local[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        out = torch.empty((x.shape[0] * h.world,) + tuple(x.shape[1:]), dtype=x.dtype, device=x.device)
        h.C.lib().symm_row_collective(1, self.buf.ptrs, h.flags.ptrs, out, x.numel(), h.rank, h.world, h.next_epoch(),
                                      h.wait_limit_s, h.abort_word)
        return out


def register_row_collectives(comm: Comm, rc: Optional[RowCollectives]) -> None:
    if rc is None:
        _ROW_COLLECTIVES.pop(id(comm), None)
    else:
        _ROW_COLLECTIVES[id(comm)] = rc


def _reduce_scatter_value(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    world, rank = comm.world_size, comm.rank
    if world == 1:
        return x
    if x.shape[0] % world:
        raise ValueError(f"{x.shape[0]} rows do not split over {world} ranks")
    rc = _ROW_COLLECTIVES.get(id(comm))
    if rc is not None:
        y = rc.reduce_scatter(x.contiguous())
        if y is not None:
            return y
    staged = x.detach().to(torch.float32).contiguous().clone()
    comm.all_reduce_sum([staged])
    n = x.shape[0] // world
    return staged[rank * n:(rank + 1) * n].to(x.dtype)


def _all_gather_value(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    world, rank = comm.world_size, comm.rank
    if world == 1:
        return x
    rc = _ROW_COLLECTIVES.get(id(comm))
    if rc is not None:
        y = rc.all_gather(x.contiguous())
        if y is not None:
            return y
    n = x.shape[0]
    staged = torch.zeros((n * world,) + tuple(x.shape[1:]), dtype=torch.float32, device=x.device)
    staged[rank * n:(rank + 1) * n] = x.detach().to(torch.float32)
    comm.all_reduce_sum([staged])          # every row is written by exactly one rank
    return staged.to(x.dtype)


def _my_rows(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    n = x.shape[0] // comm.world_size
    return x[comm.rank * n:(comm.rank + 1) * n]


class _GatherTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _all_gather_value(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _reduce_scatter_value(g.contiguous(), ctx.comm), None


class _GatherReplicated(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _all_gather_value(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _my_rows(g, ctx.comm).contiguous(), None


class _ScatterSum(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _reduce_scatter_value(x, comm)

    @staticmethod
    def backward(ctx, g):
        return _all_gather_value(g.contiguous(), ctx.comm), None


class _ShardRows(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return _my_rows(x, comm).contiguous()

    @staticmethod
    def backward(ctx, g):
        return _all_gather_value(g.contiguous(), ctx.comm), None


def all_gather_rows_value(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    """All ranks' row shards of ``x`` in rank order, outside autograd (used by backward passes)."""
    return _all_gather_value(x, comm)


def reduce_scatter_rows_value(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    """This rank's rows of the sum of ``x`` over the ranks, outside autograd (used by backward passes)."""
    return _reduce_scatter_value(x, comm)


def gather_rows_tp(x, comm):
    return x if comm.world_size == 1 else _GatherTP.apply(x, comm)


def gather_rows_replicated(x, comm):
    return x if comm.world_size == 1 else _GatherReplicated.apply(x, comm)


def scatter_rows_sum(x, comm):
    return x if comm.world_size == 1 else _ScatterSum.apply(x, comm)


def shard_rows(x, comm):
    return x if comm.world_size == 1 else _ShardRows.apply(x, comm)
