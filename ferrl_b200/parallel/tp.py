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
import torch.nn.functional as F

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


# ----------------------------------------------------------- vocabulary-sharded log-prob head
def _shard_logits(hidden, w_shard, temperature, softcap):
    z = F.linear(hidden.float(), w_shard.float())
    if softcap and softcap > 0:
        z = softcap * torch.tanh(z / softcap)
    return z / temperature


def _shard_stats_eager(hidden, w_shard, targets, temperature, softcap, col0):
    z = _shard_logits(hidden, w_shard, temperature, softcap)
    m = z.max(dim=-1).values
    s = (z - m[:, None]).exp().sum(-1)
    local = targets.long() - col0
    inside = (local >= 0) & (local < w_shard.shape[0])
    tl = torch.where(inside, z.gather(1, local.clamp(0, w_shard.shape[0] - 1)[:, None]).squeeze(1), torch.zeros_like(m))
    return torch.stack([m, s, tl], dim=1)


class _ShardedLogprob(torch.autograd.Function):
    """``log_softmax(softcap(h W^T) / T)[target]`` with the head's rows (the vocabulary) split over the tensor-parallel
    ranks: each rank scores its shard, the per-row partials (max, sum exp, target logit) are exchanged - three floats
    per row instead of a vocabulary-wide row - and every rank ends with the same log-probabilities.  Backward: each
    rank forms the hidden-state gradient of its shard from the global log-sum-exp and the partial gradients are summed
    over the ranks.  On CUDA the shard statistics and the softmax gradient come out of the head GEMM's epilogue
    (``ops.cuda``: ``logprob_head_shard_stats`` / ``logprob_head_dlogits``).  Reference: the tied, soft-capped head of
    crates/ferrl/src/gemma4.rs:1796-1804, which every tensor-parallel rank evaluates in full."""

    @staticmethod
    def forward(ctx, hidden, w_shard, targets, temperature, softcap, comm, col0):
        from .. import ops
        h = hidden.contiguous()
        t = targets.contiguous().long()
        native = ops.native(h) and h.dtype == torch.bfloat16 and w_shard.dtype == torch.bfloat16 and w_shard.shape[0] % 8 == 0 \
            and h.shape[-1] % 8 == 0 and w_shard.stride(1) == 1
        if native:
            from ..ops import cuda as C
            stats = C.lib().logprob_head_shard_stats(h, w_shard, t, float(temperature), float(softcap or 0.0), int(col0))
        else:
            stats = _shard_stats_eager(h, w_shard, t, temperature, softcap, col0)
        world, rank = comm.world_size, comm.rank
        gathered = torch.zeros(world, *stats.shape, dtype=torch.float32, device=stats.device)
        gathered[rank] = stats
        gathered = all_reduce_sum_value(gathered, comm)            # every slot is written by exactly one rank
        m = gathered[:, :, 0].max(dim=0).values
        s = (gathered[:, :, 1] * (gathered[:, :, 0] - m[None, :]).exp()).sum(0)
        lse = m + s.log()
        lp = gathered[:, :, 2].sum(0) - lse
        ctx.save_for_backward(h, w_shard, t, lse)
        ctx.meta = (float(temperature), float(softcap or 0.0), comm, int(col0), native)
        return lp

    @staticmethod
    def backward(ctx, dlp):
        h, w_shard, t, lse = ctx.saved_tensors
        temperature, softcap, comm, col0, native = ctx.meta
        coef = (-dlp).contiguous().float()
        if native:
            from ..ops import cuda as C
            N, Vs = h.shape[0], w_shard.shape[0]
            chunk = max(256, min(N, (C.LOGPROB_CHUNK_BYTES // (2 * Vs)) // 256 * 256)) if N else 1
            wt = w_shard.t().contiguous()
            dh = torch.empty_like(h)
            for s0 in range(0, N, chunk):
                dl = C.lib().logprob_head_dlogits(h[s0:s0 + chunk], w_shard, t[s0:s0 + chunk], lse[s0:s0 + chunk],
                                                  coef[s0:s0 + chunk], temperature, softcap, col0)
                dh[s0:s0 + chunk] = C.gemm(dl, wt)
                del dl
        else:
            x = F.linear(h.float(), w_shard.float())
            z, dz = x, torch.full_like(x, 1.0 / temperature)
            if softcap > 0:
                th = torch.tanh(x / softcap)
                z, dz = softcap * th, dz * (1.0 - th * th)
            z = z / temperature
            p = (z - lse[:, None]).exp()
            local = t - col0
            inside = (local >= 0) & (local < w_shard.shape[0])
            onehot = torch.zeros_like(p)
            onehot[inside, local[inside]] = 1.0
            dl = coef[:, None] * (p - onehot) * dz
            dh = (dl @ w_shard.float()).to(h.dtype)
        dh = all_reduce_sum_value(dh, comm)
        return dh, None, None, None, None, None, None


def sharded_logprob_gather(hidden, head_w, targets, temperature, softcap, comm: Comm):
    """Log-probabilities of ``targets`` from a head whose rows are split evenly over ``comm``'s ranks (this rank takes
    rows ``rank * V / world`` onward of the replicated ``head_w``; a view, nothing is copied).  ``None`` when the
    vocabulary does not split into multiples of eight rows."""
    world, rank = comm.world_size, comm.rank
    V = head_w.shape[0]
    if world == 1 or V % world or (V // world) % 8 or head_w.requires_grad:
        return None
    vs = V // world
    return _ShardedLogprob.apply(hidden, head_w[rank * vs:(rank + 1) * vs], targets, temperature, softcap, comm, rank * vs)
