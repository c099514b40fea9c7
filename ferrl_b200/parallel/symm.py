"""Symmetric peer-memory heap over NVLink (one process per GPU).

Each rank allocates the same buffers with ``cudaMalloc`` inside the native
library, exports CUDA IPC handles, exchanges them through the bootstrap
communicator (``Comm.all_gather_bytes``) and maps every peer's copy.  Kernels
receive a table of per-rank pointers and read/write peers with plain loads and
stores; ordering uses flag words in peer memory with bounded waits
(``csrc/symm/symm.cuh``).  This is the data plane that replaces the reference's
only collective, a blocking per-tensor ``ncclAllReduce``
(``crates/ferrl/src/comm/nccl/real.rs:123-189``); NCCL (``TorchDistComm``)
remains for bootstrap, host control scalars and as the measured baseline.

A kernel that reports a peer-wait timeout leaves ``kernel_status() != 0``;
``SymmHeap.check`` turns that into ``CommTimeout`` and poisons the heap so no
further peer collective is attempted (the reference's NCCL path has no timeout
at all, ``comm/nccl.rs:30-36``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..comm import Comm, CommPoisoned, CommTimeout

FLAG_SLOTS = 8
MAX_RANKS = 16
_HEAPS: dict = {}


@dataclass
class SymmBuffer:
    local: torch.Tensor        # uint8 view of this rank's copy
    ptrs: list                 # device address of every rank's copy (index = rank)

    def view(self, dtype, numel: Optional[int] = None) -> torch.Tensor:
        t = self.local.view(dtype)
        return t if numel is None else t[:numel]


class SymmHeap:
    def __init__(self, comm: Comm, device: torch.device, wait_limit_s: float = 20.0):
        from ..ops import cuda as C
        self.C = C
        self.comm, self.device = comm, device
        self.rank, self.world = comm.rank, comm.world_size
        if self.world > MAX_RANKS:
            raise ValueError(f"symmetric heap supports up to {MAX_RANKS} ranks")
        self.wait_limit_s = wait_limit_s
        self.epoch = 0
        self.poisoned: Optional[str] = None
        self._opened: list = []
        # every allocation lives as long as the heap: peers keep their mappings of it until close(), and memory that
        # was freed and handed out again under the same handle cannot be mapped a second time
        self._allocations: list = []
        with torch.cuda.device(device):
            self.flags = self.alloc(FLAG_SLOTS * MAX_RANKS * 4)
            self.abort_word = torch.zeros(1, dtype=torch.int32, device=device)
        _HEAPS[id(comm)] = self

    def alloc(self, nbytes: int) -> SymmBuffer:
        nbytes = (nbytes + 255) // 256 * 256
        lib = self.C.lib()
        with torch.cuda.device(self.device):
            local = lib.symm_alloc(nbytes)
            handle = bytes(lib.symm_handle(local).tolist())
        handles = self.comm.all_gather_bytes(handle) if self.world > 1 else [handle]
        ptrs = []
        for r, h in enumerate(handles):
            if r == self.rank:
                ptrs.append(local.data_ptr())
            else:
                with torch.cuda.device(self.device):
                    p = int(lib.symm_open(torch.tensor(list(h), dtype=torch.uint8)))
                self._opened.append(p)
                ptrs.append(p)
        if self.world > 1:
            self.comm.barrier()  # every rank has mapped every peer before anyone uses the buffer
        self._allocations.append(local)
        return SymmBuffer(local, ptrs)

    def next_epoch(self) -> int:
        """The next call number of the host-numbered kernels (all-reduce, row collectives, the data-parallel step).
        A CUDA graph would replay such a launch with the number it was captured with, and its barriers would find
        every flag already there; kernels meant for capture keep their call number on the device instead (the fused
        GEMM collectives, the expert-parallel dispatch and combine)."""
        if torch.device(self.device).type == "cuda" and torch.cuda.is_current_stream_capturing():
            raise RuntimeError("a host-numbered peer-memory collective cannot be captured in a CUDA graph")
        self.epoch += 1
        return self.epoch

    def guard(self):
        if self.poisoned is not None:
            raise CommPoisoned(self.poisoned)

    def check(self, what: str):
        """Host-side status read after a peer kernel (synchronises the stream)."""
        st = self.C.kernel_status()
        if st != 0:
            self.C.lib().reset_status()
            self.poisoned = f"{what}: kernel reported status {st} (peer wait timed out)"
            raise CommTimeout(self.poisoned)

    def all_reduce_(self, buf: SymmBuffer, out: torch.Tensor) -> torch.Tensor:
        """Sum ``buf`` (same dtype/numel as ``out``) over ranks into ``out``; one-shot, rank-ordered."""
        self.guard()
        self.C.lib().symm_all_reduce(buf.ptrs, self.flags.ptrs, out, self.rank, self.world, self.next_epoch(),
                                     self.wait_limit_s, self.abort_word)
        return out

    def close(self):
        lib = self.C.lib()
        for p in self._opened:
            lib.symm_close(p)
        self._opened = []
        self._allocations = []
        _HEAPS.pop(id(self.comm), None)


class SymmAllReducer:
    """Reusable staging buffer for activation all-reduces under tensor parallelism."""

    def __init__(self, heap: SymmHeap, max_bytes: int):
        self.heap = heap
        self.buf = heap.alloc(max_bytes)
        self.max_bytes = max_bytes

    def __call__(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        nbytes = x.numel() * x.element_size()
        if nbytes > self.max_bytes or x.dtype not in (torch.bfloat16, torch.float32) or nbytes % 16:
            return None
        stage = self.buf.local[:nbytes].view(x.dtype).view(x.shape)
        stage.copy_(x)
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
        return self.heap.all_reduce_(SymmBuffer(self.buf.local[:nbytes], self.buf.ptrs), out)


class GemmAllReducer:
    """Buffers and epochs for the fused row-parallel GEMM -> all-reduce kernel.

    ``y = sum_r (x_r W_rᵀ + t_r Bᵀ) (+ residual)`` comes out of ONE launch per rank: the
    tcgen05 GEMM's epilogue pushes each partial tile into the tile owner's staging slot over
    NVLink, the owner sums the slots in rank order and pushes the result to every peer
    while the tensor cores are already on the next tiles (``csrc/gemm/tcgen05_gemm.cu``).
    The reference issues the projection and then a blocking ``ncclAllReduce`` of the whole
    activation (``crates/ferrl/src/tensor_parallel.rs:417-510``).

    Every rank must call with the same shapes in the same order (true for lockstep
    tensor-parallel forward passes); epochs advance once per call.
    """

    BM, BN_MAX, BN_MIN = 128, 256, 64

    GATHER_MAX_ROW_TILES = 1024

    def __init__(self, heap: SymmHeap, max_rows: int, max_cols: int, nvls: bool = False, gather_cols: int = 0):
        """``nvls``: staging and receive buffers bound to NVSwitch multicast objects; the tile owner then reads the
        sum of all ranks' partials with ``multimem.ld_reduce`` and broadcasts the reduced tile with ``multimem.st``
        (raises ``parallel.nvls.NvlsUnavailable`` on every rank where the group has no multicast address)."""
        self.heap = heap
        mt = (max_rows + self.BM - 1) // self.BM
        self.max_tiles = mt * ((max_cols + self.BN_MIN - 1) // self.BN_MIN)
        npad = (max_cols + self.BN_MAX - 1) // self.BN_MAX * self.BN_MAX
        self.stage_elems = mt * self.BM * npad + heap.world * self.BM * self.BN_MAX
        self.out_elems = max_rows * max_cols
        self.mc_stage = self.mc_outbuf = 0
        if nvls:
            from .nvls import alloc_multicast
            self.stage, self.mc_stage, self._h1 = alloc_multicast(heap, self.stage_elems * 2)
            self.outbuf, self.mc_outbuf, self._h2 = alloc_multicast(heap, self.out_elems * 2)
        else:
            self.stage = heap.alloc(self.stage_elems * 2)
            self.outbuf = heap.alloc(self.out_elems * 2)
        # ready[tile][rank] and done[tile] flags, the device-resident call counter and its CTA counter, then
        # fin[rank]: the last call each peer has left (a sender waits for it before it reuses the staging slots)
        # then, for the all-gather form, agr[rank] (call number whose rows that peer has in place) and arrived[row tile]
        self.flags = heap.alloc((self.max_tiles * (MAX_RANKS + 1) + 2 + 2 * MAX_RANKS + self.GATHER_MAX_ROW_TILES) * 4)
        # all-gather -> GEMM: two [max_rows, gather_cols] input buffers used alternately (see gather_gemm)
        self.gather_elems = max_rows * gather_cols
        self.gather_bufs = [heap.alloc(self.gather_elems * 2) for _ in range(2)] if gather_cols > 0 else []
        self.gather_calls = 0
        self.flags.local.zero_()
        if torch.device(heap.device).type == "cuda":
            torch.cuda.synchronize(heap.device)
        if heap.world > 1:
            heap.comm.barrier()   # nobody signals into flags that are still being cleared
        self.epoch = 0

    def fits(self, rows: int, cols: int) -> bool:
        mt = (rows + self.BM - 1) // self.BM
        tiles = mt * ((cols + self.BN_MIN - 1) // self.BN_MIN)
        npad = (cols + self.BN_MAX - 1) // self.BN_MAX * self.BN_MAX
        return (cols % 8 == 0 and tiles <= self.max_tiles and rows * cols <= self.out_elems
                and mt * self.BM * npad + self.heap.world * self.BM * self.BN_MAX <= self.stage_elems)

    def __call__(self, a, b, a2=None, b2=None, residual=None, debug=None) -> torch.Tensor:
        self.heap.guard()
        self.epoch += 1
        h = self.heap
        return h.C.lib().gemm_allreduce(a, b, a2, b2, residual, self.stage.ptrs, self.outbuf.ptrs, self.flags.ptrs,
                                        h.rank, h.world, self.epoch, self.max_tiles, self.stage_elems,
                                        self.out_elems, h.wait_limit_s, debug, self.mc_stage, self.mc_outbuf)

    def fits_gather(self, rows: int, k: int) -> bool:
        """The all-gather form: whole 128-row tiles per rank, the gathered input fits one of the two buffers."""
        return (bool(self.gather_bufs) and rows % (self.heap.world * self.BM) == 0 and k % 8 == 0
                and rows // self.BM <= self.GATHER_MAX_ROW_TILES and rows * k <= self.gather_elems)

    def gather_gemm(self, xs: torch.Tensor, b: torch.Tensor, a2=None, b2=None):
        """``(all_gather_rows(xs) bᵀ + a2 b2ᵀ, all_gather_rows(xs))`` for this rank's ``[rows / world, k]`` block
        ``xs``: one launch whose communication warps pull the peers' blocks into a local buffer while the tensor cores
        start on the rows already here; a tile of foreign rows is loaded once its rows have arrived.  The second
        result is a view of that buffer: it is overwritten by the call after next, copy it to keep it.

        Two buffers alternate: a peer rewrites its block of a buffer two calls later, and it cannot finish the call
        in between before this rank has entered it, i.e. has finished pulling for this one."""
        h = self.heap
        h.guard()
        n, k = xs.shape
        rows = n * h.world
        buf = self.gather_bufs[self.gather_calls & 1]
        self.gather_calls += 1
        self.epoch += 1
        full = buf.local[:rows * k * 2].view(torch.bfloat16).view(rows, k)
        full[h.rank * n:(h.rank + 1) * n].copy_(xs)
        y = h.C.lib().gemm_allgather(b, a2, b2, buf.ptrs, self.flags.ptrs, h.rank, h.world, self.max_tiles, rows, k,
                                     h.wait_limit_s)
        return y, full

    def fits_scatter(self, rows: int, cols: int) -> bool:
        """The reduce-scatter form: whole 128-row tiles per rank, peer-load staging."""
        return self.mc_stage == 0 and rows % (self.heap.world * self.BM) == 0 and self.fits(rows, cols)

    def reduce_scatter(self, a, b, a2=None, b2=None) -> torch.Tensor:
        """Rows ``[rank * M / world, (rank + 1) * M / world)`` of ``sum_r (a_r b_rᵀ + a2_r b2ᵀ)``: the same kernel
        with the tile owner chosen by row block; the owner keeps the summed tile and nothing is sent back, so the
        launch moves ``(world - 1) / world`` of the partial once instead of twice."""
        self.heap.guard()
        self.epoch += 1
        h = self.heap
        return h.C.lib().gemm_allreduce(a, b, a2, b2, None, self.stage.ptrs, self.outbuf.ptrs, self.flags.ptrs,
                                        h.rank, h.world, self.epoch, self.max_tiles, self.stage_elems,
                                        self.out_elems, h.wait_limit_s, None, 0, 0, True)


_REDUCERS: dict = {}
_GEMM_REDUCERS: dict = {}


def register_gemm_all_reducer(comm: Comm, reducer: GemmAllReducer) -> None:
    _GEMM_REDUCERS[id(comm)] = reducer


def gemm_all_reducer(comm: Comm) -> Optional[GemmAllReducer]:
    return _GEMM_REDUCERS.get(id(comm))


def register_all_reducer(comm: Comm, reducer: SymmAllReducer) -> None:
    _REDUCERS[id(comm)] = reducer


def try_all_reduce(x: torch.Tensor, comm: Comm) -> Optional[torch.Tensor]:
    """Peer-memory all-reduce when a reducer is registered for ``comm``; else ``None``
    (caller falls back to the ``Comm`` seam)."""
    r = _REDUCERS.get(id(comm))
    return None if r is None else r(x)
