"""Worker for the two-process fused data-parallel test (launched by torchrun, one rank per GPU)."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run as a script from any directory
import math

import torch

from ferrl_b200.comm import TorchDistComm
from ferrl_b200.ops import eager as E
from ferrl_b200.optim import AdamWParams, FerrlAdamW
from ferrl_b200.parallel.dp import FusedDpStep
from ferrl_b200.parallel.symm import SymmAllReducer


def main():
    comm = TorchDistComm.bootstrap(timeout_s=120.0)
    dev = comm.device
    world, rank = comm.world_size, comm.rank
    shapes = [(16, 1024), (1024, 16), (5,), (100003,)]
    g0 = torch.Generator(device=dev).manual_seed(1)
    params = [torch.nn.Parameter(torch.randn(s, device=dev, generator=g0)) for s in shapes]
    ref_p = [p.detach().clone() for p in params]
    ref_m, ref_v = [torch.zeros_like(p) for p in ref_p], [torch.zeros_like(p) for p in ref_p]
    opt = FerrlAdamW(params, AdamWParams(lr=1e-2))
    fused = FusedDpStep.create(comm, params, dev)
    for step in range(1, 4):
        fused.prepare_grads()
        per_rank = []
        for r in range(world):
            gr = torch.Generator(device=dev).manual_seed(100 * step + r)
            per_rank.append([torch.randn(s, device=dev, generator=gr) for s in shapes])
        for p, g in zip(params, per_rank[rank]):
            p.grad.add_(g)
        res = fused(opt, None, 1.0, 0.0, pre_scale=1.0 / world)
        red = [sum(per_rank[r][i] for r in range(world)) / world for i in range(len(shapes))]
        norm = math.sqrt(sum(float(g.double().pow(2).sum()) for g in red))
        assert res.stepped and abs(res.grad_norm - norm) / norm < 1e-5, (res, norm)
        E.adamw_step(ref_p, red, ref_m, ref_v, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.0, step=step,
                     grad_scale=min(1.0, 1.0 / norm))
        for a, b in zip(params, ref_p):
            assert (a.detach() - b).abs().max().item() < 2e-5
    # a rank whose backward failed enters the same kernel with a large uncovered count: nobody steps,
    # every rank reads the count (this is how the trainer agrees on a backward failure without a
    # rendezvous of its own)
    before = [p.detach().clone() for p in params]
    fused.prepare_grads()
    for p in params:
        p.grad.add_(1.0)
    res = fused(opt, None, 1.0, float(2 ** 20) if rank == world - 1 else 0.0, pre_scale=1.0 / world)
    assert not res.stepped and res.uncovered >= 2 ** 20, res
    for a, b in zip(params, before):
        assert torch.equal(a.detach(), b)
    # ranks must hold bit-identical parameters
    import hashlib
    digest = hashlib.sha256(b"".join(p.detach().cpu().numpy().tobytes() for p in params)).digest()
    comm.require_consensus(digest, "parameters after fused steps")
    red = SymmAllReducer(fused.heap, 1 << 22)
    x = (torch.arange(4096 * 64, device=dev, dtype=torch.float32).view(4096, 64) % 13 + rank).to(torch.bfloat16)
    y = red(x)
    want = sum((torch.arange(4096 * 64, device=dev, dtype=torch.float32).view(4096, 64) % 13 + r) for r in range(world))
    assert torch.equal(y.float(), want.to(torch.bfloat16).float())
    fused.heap.check("all-reduce")
    comm.barrier()
    if rank == 0:
        print("DP_STEP_PASS")
    import torch.distributed as dist
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
