"""Activation all-reduce through NVSwitch multicast (NVLS).

The symmetric buffer comes from ``torch.distributed._symmetric_memory`` (CUDA virtual-memory allocation
bound to a multicast object, handles exchanged through the process group's store); the arithmetic is
this package's kernel (``csrc/symm/nvls_all_reduce.cu``): ``multimem.ld_reduce`` lets the switch form
the sum, ``multimem.st`` broadcasts it, two shots so that every rank ends with the same bits.  The
barriers are the flag words of the ``SymmHeap`` (plain peer stores with bounded waits), so a wait that
runs out is reported the same way as in the other peer-memory kernels.

Opt-in (``ParallelRuntime.create(..., nvls=True)`` or ``FERRL_NVLS=1``): a process that dies while its
memory is bound to a multicast object can fault its peers' GPUs, so the default data plane stays on
plain peer loads and stores, and failure tests never run with this reducer.  The reference has no
counterpart: its tensor-parallel reduce is a blocking ``ncclAllReduce`` per activation
(``crates/ferrl/src/tensor_parallel.rs:417-510``).
"""
from __future__ import annotations

from typing import Optional

import torch

from .symm import SymmHeap


class NvlsUnavailable(RuntimeError):
    """No multicast address for this group (no NVSwitch, no driver support, or not one process per GPU)."""


def alloc_multicast(heap: SymmHeap, nbytes: int, group=None):
    """A symmetric buffer bound to an NVSwitch multicast object: ``(SymmBuffer, multicast address, handle)``.
    Collective over the process group; raises ``NvlsUnavailable`` on every rank if any rank has no address."""
    import torch.distributed as dist
    from .symm import SymmBuffer
    try:
        import torch.distributed._symmetric_memory as symm_mem
    except ImportError as e:  # pragma: no cover - depends on the torch build
        raise NvlsUnavailable(f"torch has no symmetric-memory module: {e}") from e
    if not dist.is_initialized():
        raise NvlsUnavailable("torch.distributed is not initialised")
    group = group if group is not None else dist.group.WORLD
    nbytes = (int(nbytes) + 255) // 256 * 256
    failure, mc, buf, handle, ptrs = None, 0, None, None, []
    try:
        with torch.cuda.device(heap.device):
            buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=heap.device)
            handle = symm_mem.rendezvous(buf, group)
        mc = int(getattr(handle, "multicast_ptr", 0) or 0)
        ptrs = [int(p) for p in handle.buffer_ptrs]
    except Exception as e:  # noqa: BLE001 - any allocation / rendezvous failure means "not available here"
        failure = e
    ok = heap.comm.all_reduce_scalar_sum(1.0 if mc and len(ptrs) == heap.world else 0.0)
    if ok != heap.world:
        raise NvlsUnavailable(f"no multicast address on {heap.world - int(ok)} rank(s)" + (f": {failure}" if failure is not None else ""))
    return SymmBuffer(buf, ptrs), mc, handle


class NvlsAllReducer:
    def __init__(self, heap: SymmHeap, max_bytes: int, group=None):
        import torch.distributed as dist
        try:
            import torch.distributed._symmetric_memory as symm_mem
        except ImportError as e:  # pragma: no cover - depends on the torch build
            raise NvlsUnavailable(f"torch has no symmetric-memory module: {e}") from e
        if not dist.is_initialized():
            raise NvlsUnavailable("torch.distributed is not initialised")
        self.heap = heap
        self.world, self.rank = heap.world, heap.rank
        unit = 16 * self.world
        self.max_bytes = (int(max_bytes) + unit - 1) // unit * unit
        group = group if group is not None else dist.group.WORLD
        failure = None
        self.mc_ptr = 0
        try:
            with torch.cuda.device(heap.device):
                self.buf = symm_mem.empty(self.max_bytes, dtype=torch.uint8, device=heap.device)
                self.handle = symm_mem.rendezvous(self.buf, group)
            self.mc_ptr = int(getattr(self.handle, "multicast_ptr", 0) or 0)
        except Exception as e:  # noqa: BLE001 - any allocation / rendezvous failure means "not available here"
            failure = e
        # all ranks must agree, or some would enter the kernel's barrier alone
        ok = heap.comm.all_reduce_scalar_sum(1.0 if self.mc_ptr else 0.0)
        if ok != self.world:
            raise NvlsUnavailable(f"no multicast address on {self.world - int(ok)} rank(s)"
                                  + (f": {failure}" if failure is not None else ""))

    def __call__(self, x: torch.Tensor) -> Optional[torch.Tensor]:
        nbytes = x.numel() * x.element_size()
        if nbytes == 0 or nbytes > self.max_bytes or x.dtype not in (torch.bfloat16, torch.float32) \
                or nbytes % (16 * self.world):
            return None
        self.heap.guard()
        self.buf[:nbytes].view(x.dtype).view(x.shape).copy_(x)
        out = torch.empty_like(x, memory_format=torch.contiguous_format)
        self.heap.C.lib().nvls_all_reduce(self.mc_ptr, self.buf, self.heap.flags.ptrs, out, self.rank, self.world,
                                          self.heap.next_epoch(), self.heap.wait_limit_s, self.heap.abort_word)
        return out
