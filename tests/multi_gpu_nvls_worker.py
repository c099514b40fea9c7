"""Worker for the multi-process NVLS all-reduce test (torchrun, one rank per GPU).

The in-switch all-reduce (``multimem.ld_reduce`` / ``multimem.st``) against the plain peer-load all-reduce of
the symmetric heap on several shapes and repeated calls: same sums up to the order of the additions,
bit-identical on every rank.  Prints device timings of both and of NCCL for a 64 MB bf16 activation.
Prints ``NVLS_UNAVAILABLE`` and passes where the group has no multicast address.
Every rank leaves only after a final barrier, with no kernel in flight.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run as a script from any directory
import hashlib

import torch
import torch.distributed as dist

from ferrl_b200.comm import TorchDistComm
from ferrl_b200.parallel.nvls import NvlsAllReducer, NvlsUnavailable
from ferrl_b200.parallel.symm import SymmAllReducer, SymmHeap


def _time(fn, iters=20):
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    dist.barrier()
    s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    s.record()
    for _ in range(iters):
        fn()
    e.record()
    torch.cuda.synchronize()
    t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t)


def main():
    comm = TorchDistComm.bootstrap(timeout_s=120.0)
    dev, rank, world = comm.device, comm.rank, comm.world_size
    heap = SymmHeap(comm, dev, wait_limit_s=20.0)
    max_bytes = 8192 * 4096 * 2
    plain = SymmAllReducer(heap, max_bytes)
    try:
        fast = NvlsAllReducer(heap, max_bytes)
    except NvlsUnavailable as e:
        comm.barrier()
        if rank == 0:
            print(f"NVLS_UNAVAILABLE {e}")
        dist.destroy_process_group()
        return 0
    failed = None
    try:
        _checks(comm, heap, plain, fast, dev, rank, world)
    except BaseException as e:  # noqa: BLE001 - no rank may leave while its peers still hold the multicast binding
        failed = f"{type(e).__name__}: {e}"
    torch.cuda.synchronize()
    flags = comm.all_gather_bytes((failed or "").encode())
    if rank == 0:
        bad = [f"rank {r}: {b.decode()}" for r, b in enumerate(flags) if b]
        print("NVLS_FAIL " + " | ".join(bad) if bad else "NVLS_PASS")
    comm.barrier()
    dist.destroy_process_group()
    return 1 if any(flags) else 0


def _checks(comm, heap, plain, fast, dev, rank, world):
    for it, (shape, dtype) in enumerate([((128, 4096), torch.bfloat16), ((4096, 5376), torch.bfloat16), ((777 * world, 64), torch.float32),
                                         ((128, 4096), torch.bfloat16), ((8192, 4096), torch.bfloat16)]):
        g = torch.Generator(device=dev).manual_seed(100 * it + rank)
        x = torch.randn(shape, device=dev, generator=g).to(dtype)
        y = fast(x)
        assert y is not None, shape
        heap.check("nvls all-reduce")
        ref = plain(x)
        heap.check("plain all-reduce")
        # exact sum in fp64 from every rank's input
        parts = [torch.randn(shape, device=dev, generator=torch.Generator(device=dev).manual_seed(100 * it + r)).to(dtype).double()
                 for r in range(world)]
        exact = sum(parts)
        tol = (2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -22) * float(exact.abs().max()) * 2
        assert float((y.double() - exact).abs().max()) <= tol, (shape, float((y.double() - exact).abs().max()), tol)
        assert float((y.double() - ref.double()).abs().max()) <= tol
        digest = hashlib.sha256(y.cpu().view(torch.uint8).numpy().tobytes()).digest()
        assert len(set(comm.all_gather_bytes(digest))) == 1, f"ranks hold different results for case {it}"
    assert fast(torch.zeros(3, 5, device=dev)) is None          # not a multiple of 16 * world bytes: declined
    x = torch.randn(8192, 4096, device=dev).to(torch.bfloat16)
    t_fast = _time(lambda: fast(x))
    t_plain = _time(lambda: plain(x))
    xn = x.clone()
    t_nccl = _time(lambda: dist.all_reduce(xn))
    heap.check("timing")
    if rank == 0:
        gb = x.numel() * 2 / 1e9
        print(f"NVLS_TIMING world={world} bytes={x.numel() * 2} nvls_ms={t_fast:.4f} peer_load_ms={t_plain:.4f} nccl_ms={t_nccl:.4f} "
              f"nvls_algbw_GBps={gb / (t_fast * 1e-3):.0f}")


if __name__ == "__main__":
    sys.exit(main())
