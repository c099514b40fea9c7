"""Gradient all-reduce micro-benchmark: the fused peer-memory step against per-tensor NCCL.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 8 --master-addr 127.0.0.1 \
        examples/dp_allreduce.py [--tensors 504] [--iters 20]

Builds Qwen3-8B's LoRA r16 adapter set (504 tensors, 43.6 M fp32 values), fills the gradients
and times (a) ``FusedDpStep`` - reduce-scatter + scale + global norm + clip + AdamW in one
cooperative kernel over NVLink peer memory - and (b) the reference's shape: one NCCL all-reduce
per tensor, then norm, clip and AdamW.  Device time, max over ranks.  Counterpart of
``crates/ferrl/examples/nccl_dp_allreduce.rs``.
"""
import argparse
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))

import torch  # noqa: E402
import torch.distributed as dist  # noqa: E402

from ferrl_b200.comm import TorchDistComm  # noqa: E402
from ferrl_b200.optim import AdamWParams, FerrlAdamW  # noqa: E402
from ferrl_b200.parallel.dp import FusedDpStep  # noqa: E402


def timed(fn, iters):
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


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--tensors", type=int, default=504)
    ap.add_argument("--iters", type=int, default=20)
    args = ap.parse_args(argv)
    comm = TorchDistComm.bootstrap(timeout_s=300.0)
    dev = comm.device
    shapes = ([(16, 4096), (6144, 16), (16, 4096), (4096, 16), (16, 4096), (24576, 16), (16, 12288), (4096, 16)] * 64)[:args.tensors]
    params = [torch.nn.Parameter(torch.zeros(s, device=dev)) for s in shapes]
    opt = FerrlAdamW(params, AdamWParams(lr=1e-5))
    fused = FusedDpStep.create(comm, params, dev)

    def fused_step():
        fused.prepare_grads()
        for p in params:
            p.grad.fill_(1e-3)
        fused(opt, None, 1.0, 0.0, pre_scale=1.0 / comm.world_size)

    def nccl_step():
        for p in params:
            if p.grad is None:
                p.grad = torch.zeros_like(p)
            p.grad.fill_(1e-3)
        for p in params:
            dist.all_reduce(p.grad)                      # one blocking collective per tensor, as the reference does
        inv = 1.0 / comm.world_size
        norm = float(torch.sqrt(sum((p.grad * inv).double().pow(2).sum() for p in params)))   # host-synchronised norm
        opt.step([p.grad for p in params], grad_scale=inv * min(1.0, 1.0 / max(norm, 1e-12)))

    t_fused = timed(fused_step, args.iters)
    fused.heap.check("fused step")
    t_nccl = timed(nccl_step, args.iters)
    if comm.rank == 0:
        n = sum(p.numel() for p in params)
        print(f"world {comm.world_size}: {len(params)} tensors, {n / 1e6:.1f} M values; fused {t_fused:.3f} ms, "
              f"per-tensor NCCL + norm + AdamW {t_nccl:.3f} ms")
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
