"""Worker for the multi-process expert-parallel test (torchrun, one rank per GPU): experts sharded
over ranks through the peer-memory dispatch/combine kernels must give every rank the result of the
local plan over all experts, forward and backward, on repeated calls."""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run as a script from any directory

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
    # the decode step is replayed from a CUDA graph: the kernels' barriers must use a fresh call number on every
    # replay (it lives on the device), so replays with new inputs must keep matching the local plan
    Td = 128
    xs_ = torch.zeros(Td, H, device=dev, dtype=torch.bfloat16)
    lg_ = torch.zeros(Td, E, device=dev)
    gu_l, dn_l = gate_up[lo:hi].contiguous(), down[lo:hi].contiguous()

    def step():
        with torch.no_grad():
            sc_, idx_, cnt_, _ = C.moe_route(lg_, k, True)
            return rt.experts(xs_, sc_, idx_, cnt_, gu_l, dn_l, "silu")
    step()
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y_static = step()
    for rep in range(4):
        xs_.copy_(torch.randn(Td, H, device=dev, generator=gl).to(torch.bfloat16))
        lg_.copy_(torch.randn(Td, E, device=dev, generator=gl))
        graph.replay()
        with torch.no_grad():
            sc_, idx_, cnt_, _ = C.moe_route(lg_, k, True)
            want = C.moe_experts(xs_, sc_, idx_, cnt_, gate_up, down, "silu")
        torch.cuda.synchronize()
        heap.check("expert-parallel graph replay")
        assert torch.equal(y_static, want), (rep, float((y_static.float() - want.float()).abs().max()))
    comm.barrier()
    if rank == 0:
        print("EP_GRAPH_REPLAY_PASS")
    # timing at the hybrid-MoE benchmark's layer shape: 128 experts top-8, hidden 2048, expert FFN 768
    if world in (2, 4, 8):
        T2, E2, k2, H2, I2 = 8192, 128, 8, 2048, 768
        rt2 = EpRuntime(heap, E2, H2, T2, k2, capacity_factor=2.0)
        gu2 = (torch.randn(E2 // world, 2 * I2, H2, device=dev, generator=g) / H2 ** 0.5).to(torch.bfloat16)
        dn2 = (torch.randn(E2 // world, H2, I2, device=dev, generator=g) / I2 ** 0.5).to(torch.bfloat16)
        x2 = torch.randn(T2, H2, device=dev, generator=gl).to(torch.bfloat16)
        sc2, idx2, cnt2, _ = C.moe_route(torch.randn(T2, E2, device=dev, generator=gl), k2, True)   # router logits N(0,1)

        def run():
            with torch.no_grad():
                return rt2.experts(x2, sc2, idx2, cnt2, gu2, dn2, "silu")
        for _ in range(3):
            run()
        torch.cuda.synchronize()
        dist.barrier()
        s_, e_ = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s_.record()
        for _ in range(10):
            run()
        e_.record()
        torch.cuda.synchronize()
        heap.check("expert-parallel timing")
        tt = torch.tensor([s_.elapsed_time(e_) / 10], device=dev)
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
        if rank == 0:
            sent = T2 * k2 * H2 * 2 * (world - 1) / world          # bytes a rank pushes out in dispatch (and pulls back in combine)
            flops = 2 * T2 * k2 * H2 * 3 * I2                       # gate_up + down per routed row, per rank's tokens
            print(f"EP_TIMING world={world} tokens/rank={T2} ms={float(tt):.4f} dispatch_bytes_out={sent / 1e6:.1f}MB "
                  f"combine_bytes_in={sent / 1e6:.1f}MB expert_flops/rank={flops / 1e9:.1f}G")
    comm.barrier()
    if rank == 0:
        print("EP_PASS")
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
