"""Worker for the multi-process expert-parallel test (torchrun, one rank per GPU): experts sharded
over ranks through the peer-memory dispatch/combine kernels must give every rank the result of the
local plan over all experts, forward and backward, on repeated calls."""
import sys

import torch
import torch.distributed as dist

from ferrl_b200.comm import TorchDistComm
from ferrl_b200.ops import cuda as C
from ferrl_b200.parallel.ep import EpRuntime
from ferrl_b200.parallel.symm import SymmHeap


def main():
    comm = TorchDistComm.bootstrap(timeout_s=120.0)
    dev, world, rank = comm.device, comm.world_size, comm.rank
    heap = SymmHeap(comm, dev, wait_limit_s=20.0)
    T, E, k, H, I = 900, 16, 4, 256, 128
    rt = EpRuntime(heap, E, H, T, k, capacity_factor=float(world))
    g = torch.Generator(device=dev).manual_seed(3)                 # identical experts on every rank
    gate_up = (torch.randn(E, 2 * I, H, device=dev, generator=g) / H ** 0.5).to(torch.bfloat16)
    down = (torch.randn(E, H, I, device=dev, generator=g) / I ** 0.5).to(torch.bfloat16)
    lo, hi = rank * (E // world), (rank + 1) * (E // world)
    gl = torch.Generator(device=dev).manual_seed(100 + rank)       # different tokens on every rank
    for rep in range(3):
        x = torch.randn(T - 7 * rank, H, device=dev, generator=gl).to(torch.bfloat16)
        scores, idx, counts, _ = C.moe_route(torch.randn(x.shape[0], E, device=dev, generator=gl), k, True)
        dy = torch.randn(x.shape[0], H, device=dev, generator=gl).to(torch.bfloat16)
        res = []
        for sharded in (False, True):
            xx = x.detach().clone().requires_grad_(True)
            ss = scores.detach().clone().requires_grad_(True)
            if sharded:
                y = rt.experts(xx, ss, idx, counts, gate_up[lo:hi].contiguous(), down[lo:hi].contiguous(), "silu")
            else:
                y = C.moe_experts(xx, ss, idx, counts, gate_up, down, "silu")
            y.backward(dy)
            res.append((y.detach(), xx.grad, ss.grad))
        torch.cuda.synchronize()
        heap.check("expert-parallel step")
        for a, b in zip(res[0], res[1]):
            assert torch.equal(a, b), (rep, float((a.float() - b.float()).abs().max()))
    comm.barrier()
    if rank == 0:
        print("EP_PASS")
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
