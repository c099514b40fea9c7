"""Per-launch wiring of the peer-memory data plane into the model path.

A launch with ``tensor_parallel.enabled`` or ``expert_parallel.enabled`` gets one
``ParallelRuntime``: it owns the symmetric heap, registers the fused GEMM -> all-reduce kernel and
the activation all-reducer for the tensor-parallel communicator (so ``FusedLoraLinear.forward_reduce``
and ``reduce_from_tp`` reach the kernels instead of the NCCL ``Comm`` seam), and installs the
expert-parallel context whose dispatch/combine kernels the MoE blocks call.  The trainer calls
``check`` at a step boundary: a bounded peer wait that ran out surfaces there as ``CommTimeout``
and poisons the heap, instead of letting the step continue on an unfinished tile.

The reference reduces after every row-parallel projection with a blocking NCCL all-reduce
(``crates/ferrl/src/tensor_parallel.rs:417-510``) and has no expert parallelism
(``crates/ferrl/src/moe.rs:110-158``).
"""
from __future__ import annotations

import os
from dataclasses import dataclass, field
from typing import Callable, Optional

import torch

from ..comm import Comm


def gloo_all_to_all_rows(comm: Comm):
    """Row all-to-all for expert parallelism over the host control plane (CPU ranks, tests).
    ``rows`` sorted by destination rank, ``per_rank[r]`` rows go to rank ``r``."""
    import io

    def a2a(rows, per_rank, expert_counts):
        world, me = comm.world_size, comm.rank
        send = [int(v) for v in per_rank.tolist()]
        offs = [0]
        for n in send:
            offs.append(offs[-1] + n)
        buf = io.BytesIO()
        torch.save({"rows": [rows[offs[r]:offs[r + 1]].detach().cpu() for r in range(world)],
                    "ec": None if expert_counts is None else expert_counts.detach().cpu()}, buf)
        blobs = comm.all_gather_bytes(buf.getvalue())
        got = [torch.load(io.BytesIO(b)) for b in blobs]
        parts = [g["rows"][me].to(rows.device) for g in got]
        recv = torch.cat(parts, 0) if parts else rows.new_empty((0, rows.shape[1]))
        recv_n = torch.tensor([p.shape[0] for p in parts], dtype=torch.long, device=rows.device)
        rec = None
        if expert_counts is not None:
            rec = torch.stack([g["ec"][me].long() for g in got]).to(rows.device)
        return recv, recv_n, rec
    return a2a


class _FirstOf:
    """An activation all-reducer that tries ``first`` and falls back to ``second`` for inputs it declines."""

    def __init__(self, first, second):
        self.first, self.second = first, second

    def __call__(self, x):
        y = self.first(x)
        return y if y is not None else self.second(x)


@dataclass
class ParallelRuntime:
    comm: Comm
    heap: Optional[object] = None
    gemm_reducer: Optional[object] = None
    all_reducer: Optional[object] = None
    ep_context: Optional[object] = None
    row_collectives: Optional[object] = None
    notes: list = field(default_factory=list)

    @classmethod
    def create(cls, comm: Comm, device, *, tensor_parallel: bool = False, hidden: int = 0, max_rows: int = 0,
               expert_parallel: Optional[dict] = None, heap_factory: Optional[Callable] = None,
               wait_limit_s: float = 20.0, nvls: Optional[bool] = None, sequence_parallel: bool = False) -> "ParallelRuntime":
        """``max_rows``: most activation rows (tokens) one forward call carries; ``hidden``: model width.
        ``sequence_parallel``: also allocate the input buffers of the fused all-gather -> GEMM kernel.
        ``expert_parallel``: ``{num_experts, hidden, max_tokens, top_k, capacity_factor}``."""
        from . import ep as EP
        from . import symm
        rt = cls(comm)
        dev = torch.device(device)
        on_gpu = dev.type == "cuda" and comm.world_size > 1
        if on_gpu or heap_factory is not None:
            rt.heap = (heap_factory or symm.SymmHeap)(comm, dev, wait_limit_s)
        if tensor_parallel and comm.world_size > 1 and rt.heap is not None:
            rows = max(int(max_rows), 128)
            gcols = int(hidden) if sequence_parallel and on_gpu else 0
            plain = symm.SymmAllReducer(rt.heap, rows * int(hidden) * 4)
            rt.all_reducer = plain
            how = "peer-memory"
            if (os.environ.get("FERRL_NVLS") == "1" if nvls is None else nvls) and on_gpu:
                # in-switch reduction, in the fused projection kernel and for the plain activation all-reduce
                # (inputs the latter does not take fall back to peer loads)
                from .nvls import NvlsAllReducer, NvlsUnavailable
                try:
                    rt.gemm_reducer = symm.GemmAllReducer(rt.heap, rows, int(hidden), nvls=True, gather_cols=gcols)
                    fast = NvlsAllReducer(rt.heap, rows * int(hidden) * 4)
                    rt.all_reducer = _FirstOf(fast, plain)
                    how = "NVLS multimem"
                except NvlsUnavailable as e:
                    rt.gemm_reducer = None
                    rt.notes.append(f"nvls unavailable: {e}")
            if rt.gemm_reducer is None:
                rt.gemm_reducer = symm.GemmAllReducer(rt.heap, rows, int(hidden), gather_cols=gcols)
            symm.register_gemm_all_reducer(comm, rt.gemm_reducer)
            symm.register_all_reducer(comm, rt.all_reducer)
            if on_gpu:
                # reduce-scatter / all-gather over the token rows for sequence-sharded models (parallel/sp.py)
                from . import sp
                rt.row_collectives = sp.RowCollectives(rt.heap, rows * int(hidden) * 4)
                sp.register_row_collectives(comm, rt.row_collectives)
            rt.notes.append(f"tp: fused gemm->all-reduce + {how} activation all-reduce")
        if expert_parallel is not None and comm.world_size > 1:
            e = expert_parallel
            runtime = None
            if rt.heap is not None and on_gpu:
                runtime = EP.EpRuntime(rt.heap, e["num_experts"], e["hidden"], e["max_tokens"], e["top_k"],
                                       e.get("capacity_factor", 2.0))
            rt.ep_context = EP.EpContext(comm.rank, comm.world_size,
                                         all_to_all_rows=None if runtime is not None else gloo_all_to_all_rows(comm),
                                         runtime=runtime)
            EP.install(rt.ep_context)
            rt.notes.append("ep: peer-memory dispatch/combine" if runtime is not None else "ep: host all-to-all")
        return rt

    def check(self, what: str) -> None:
        """Read the kernels' status word; raises ``CommTimeout`` (and poisons the heap) when a peer wait ran out."""
        if self.heap is not None:
            self.heap.check(what)

    def close(self) -> None:
        from . import ep as EP
        from . import symm
        if self.ep_context is not None and EP.current() is self.ep_context:
            EP.install(None)
        symm._GEMM_REDUCERS.pop(id(self.comm), None)
        symm._REDUCERS.pop(id(self.comm), None)
        if self.row_collectives is not None:
            from . import sp
            sp.register_row_collectives(self.comm, None)
        if self.heap is not None and hasattr(self.heap, "close"):
            self.heap.close()
