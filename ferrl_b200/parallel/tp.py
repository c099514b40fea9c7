"""Tensor-parallel planning and the autograd seams around the collectives.

Megatron layout, as in the reference (``crates/ferrl/src/tensor_parallel.rs``
``:82-192`` plan, ``:301-322`` column/row linears, ``:417-510`` reductions):
q/k/v/gate/up are column-parallel (output rows split, heads and kv-heads split
evenly), o/down are row-parallel (input columns split) and produce partial sums
that are all-reduced.  Embeddings, norms, the LM head and the LoRA masters are
replicated.

The two autograd operators are the classic pair:

* ``copy_to_tp``      forward identity, backward sum-all-reduce of the cotangent
* ``reduce_from_tp``  forward sum-all-reduce, backward identity

On GPUs ``reduce_from_tp`` is not issued as a separate collective: the
row-parallel projection calls the all-reduce mode of the GEMM kernel
(``csrc/gemm/tcgen05_gemm.cu``), which pushes partial tiles over NVLink while later tiles are
still on the tensor cores.  The functions here are the CPU/``Comm`` form used
by lockstep tests and as the NCCL baseline.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..comm import Comm, CommConfigError


@dataclass(frozen=True)
class ShardRange:
    start: int
    len: int

    @property
    def end(self) -> int:
        return self.start + self.len


@dataclass(frozen=True)
class TensorParallelPlan:
    rank: int
    world: int
    num_heads: int
    num_kv_heads: int
    intermediate: int

    @staticmethod
    def new(rank: int, world: int, num_heads: int, num_kv_heads: int, intermediate: int) -> "TensorParallelPlan":
        if world < 1 or rank < 0 or rank >= world:
            raise CommConfigError(f"tensor-parallel rank {rank} outside world {world}")
        for name, v in (("attention heads", num_heads), ("kv heads", num_kv_heads),
                        ("intermediate size", intermediate)):
            if v % world:
                raise CommConfigError(f"{name} ({v}) must divide evenly over {world} tensor-parallel ranks")
        return TensorParallelPlan(rank, world, num_heads, num_kv_heads, intermediate)

    @property
    def local_heads(self) -> int:
        return self.num_heads // self.world

    @property
    def local_kv_heads(self) -> int:
        return self.num_kv_heads // self.world

    @property
    def local_intermediate(self) -> int:
        return self.intermediate // self.world

    def shard(self, total: int) -> ShardRange:
        per = total // self.world
        return ShardRange(self.rank * per, per)


class _CopyToTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        ctx.comm = comm
        return x.view_as(x)

    @staticmethod
    def backward(ctx, g):
        return all_reduce_sum_value(g, ctx.comm), None


class _ReduceFromTP(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, comm):
        return all_reduce_sum_value(x, comm)

    @staticmethod
    def backward(ctx, g):
        return g, None


def all_reduce_sum_value(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    """Sum ``x`` over ranks.  bf16 payloads are staged through float32 for the
    ``Comm`` seam (f32/f64 gate) and cast back."""
    if comm.world_size == 1:
        return x
    from . import symm
    fused = symm.try_all_reduce(x, comm)      # None unless a peer-memory reducer is registered for this communicator
    if fused is not None:
        return fused
    staged = x.detach().to(torch.float32).contiguous().clone()
    comm.all_reduce_sum([staged])
    return staged.to(x.dtype)


def copy_to_tp(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    if comm.world_size == 1:
        return x
    return _CopyToTP.apply(x, comm)


def reduce_from_tp(x: torch.Tensor, comm: Comm) -> torch.Tensor:
    if comm.world_size == 1:
        return x
    return _ReduceFromTP.apply(x, comm)
