"""Worker for the multi-process tensor-parallel test (torchrun, one rank per GPU).

1. the fused GEMM -> all-reduce kernel against an fp32 reference and against the NCCL path,
   over several shapes and repeated calls (epochs, buffer reuse), bit-identical on every rank;
2. a tensor-parallel dense layer stack: forward and adapter gradients with the fused kernel
   equal the ones with a separate all-reduce.
Prints device timings of fused vs. GEMM + NCCL all-reduce for one training-shaped problem.
"""
import os
import sys

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))   # run as a script from any directory
import hashlib

import torch
import torch.distributed as dist

from ferrl_b200.comm import TorchDistComm
from ferrl_b200.ops import cuda as C
from ferrl_b200.parallel.symm import GemmAllReducer, SymmHeap, register_gemm_all_reducer


def _time(fn, iters=10):
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


def _check_reducer(comm, heap, red, dev, world, rank, what):
    for i, (M, N, K, use_res, use_lora) in enumerate([(300, 512, 256, False, False), (1000, 4096, 1024, True, True),
                                                      (128, 4096, 2048, True, False), (8192, 4096, 2048, True, True),
                                                      (300, 512, 256, True, False)]):
        parts, want = [], None
        gen = torch.Generator(device=dev).manual_seed(17 + i)
        b2 = (torch.randn(N, 16, device=dev, generator=gen) * 0.1).to(torch.bfloat16) if use_lora else None
        residual = torch.randn(M, N, device=dev, generator=gen).to(torch.bfloat16) if use_res else None
        mine = None
        for r in range(world):
            a = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            b = (torch.randn(N, K, device=dev, generator=gen) / K ** 0.5).to(torch.bfloat16)
            t2 = torch.randn(M, 16, device=dev, generator=gen).to(torch.bfloat16) if use_lora else None
            p = a.float() @ b.float().t()
            if use_lora:
                p = p + t2.float() @ b2.float().t()
            parts.append(p.to(torch.bfloat16).float())
            if r == rank:
                mine = (a, b, t2)
        want = sum(parts) + (residual.float() if use_res else 0.0)
        for rep in range(3):
            y = red(mine[0], mine[1], mine[2], b2, residual)
            torch.cuda.synchronize()
            heap.check("fused gemm all-reduce")
            err = float((y.float() - want).abs().max())
            assert err <= 0.02 * float(want.abs().max()), (M, N, K, rep, err)
            digest = hashlib.sha256(y.cpu().view(torch.int16).numpy().tobytes()).digest()
            comm.require_consensus(digest, f"{what} output {M}x{N}x{K} rep {rep}")


def _check_reduce_scatter(comm, heap, red, dev, world, rank):
    """Reduce-scatter form of the fused kernel: this rank's rows must equal, bit for bit, the same rows of the
    all-reduce form (both sum the partials in rank order), also when the two forms alternate back to back."""
    for i, (M, N, K, use_lora) in enumerate([(world * 128, 512, 256, False), (world * 512, 4096, 1024, True),
                                             (8192, 4096, 2048, True)]):
        gen = torch.Generator(device=dev).manual_seed(101 + i)
        b2 = (torch.randn(N, 16, device=dev, generator=gen) * 0.1).to(torch.bfloat16) if use_lora else None
        mine = None
        for r in range(world):
            a = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)
            b = (torch.randn(N, K, device=dev, generator=gen) / K ** 0.5).to(torch.bfloat16)
            t2 = torch.randn(M, 16, device=dev, generator=gen).to(torch.bfloat16) if use_lora else None
            if r == rank:
                mine = (a, b, t2)
        assert red.fits_scatter(M, N)
        n = M // world
        for rep in range(4):
            full = red(mine[0], mine[1], mine[2], b2, None)
            part = red.reduce_scatter(mine[0], mine[1], mine[2], b2)
            part2 = red.reduce_scatter(mine[0], mine[1], mine[2], b2)
            torch.cuda.synchronize()
            heap.check("fused gemm reduce-scatter")
            assert part.shape == (n, N)
            assert torch.equal(part, full[rank * n:(rank + 1) * n]), (M, N, K, rep)
            assert torch.equal(part2, part), (M, N, K, rep)
    comm.barrier()
    if rank == 0:
        print("TP_REDUCE_SCATTER_PASS")


def _check_gather_gemm(comm, heap, dev, world, rank):
    """All-gather -> GEMM in one launch against gather-then-GEMM: fresh inputs every call (a tile loaded before its rows
    arrived would show the previous call's data), shapes whose K is and is not a multiple of the 256-column pull unit."""
    red = GemmAllReducer(heap, 8192, 4096, gather_cols=5376)
    for i, (M, N, K, use_lora) in enumerate([(world * 128, 512, 256, False), (world * 512, 1024, 264, True),
                                             (world * 1024, 2048, 5376, True), (8192, 4096, 2048, False)]):
        assert red.fits_gather(M, K)
        n = M // world
        for rep in range(4):
            gen = torch.Generator(device=dev).manual_seed(4000 + 100 * i + rep)
            x = torch.randn(M, K, device=dev, generator=gen).to(torch.bfloat16)          # same on every rank
            b = (torch.randn(N, K, device=dev, generator=torch.Generator(device=dev).manual_seed(77 + rank)) / K ** 0.5).to(torch.bfloat16)
            t2 = torch.randn(M, 16, device=dev, generator=gen).to(torch.bfloat16) if use_lora else None
            b2 = (torch.randn(N, 16, device=dev, generator=gen) * 0.1).to(torch.bfloat16) if use_lora else None
            y, full = red.gather_gemm(x[rank * n:(rank + 1) * n].contiguous(), b, t2, b2)
            torch.cuda.synchronize()
            heap.check("fused all-gather gemm")
            assert torch.equal(full, x), (M, N, K, rep)
            want = C.gemm(x, b, t2, b2)
            err = float((y.float() - want.float()).abs().max())
            assert err <= 2.0 ** -7 * float(want.float().abs().max()), (M, N, K, rep, err)
    M, K, N = 8192, 4096, 12288 // world
    x = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    n = M // world
    xs = x[rank * n:(rank + 1) * n].contiguous()
    t_fused = _time(lambda: red.gather_gemm(xs, b))
    full = torch.empty(M, K, device=dev, dtype=torch.bfloat16)

    def unfused():
        dist.all_gather_into_tensor(full, xs)
        return C.gemm(full, b)
    t_nccl = _time(unfused)
    t_gemm = _time(lambda: C.gemm(x, b))
    heap.check("all-gather gemm timing")
    comm.barrier()
    if rank == 0:
        print(f"TP_AG_TIMING world={world} M={M} N={N} K={K} fused_all_gather_gemm_ms={t_fused:.4f} "
              f"nccl_all_gather_gemm_ms={t_nccl:.4f} gemm_only_ms={t_gemm:.4f}")
        print("TP_ALL_GATHER_GEMM_PASS")


def _nvls_variant(comm, heap, dev, world, rank, a, b, res, t_nccl):
    """The in-switch form of the same kernel (FERRL_TEST_NVLS=1): same checks, its own timing line.  No rank
    leaves this function before all have finished with the multicast-bound buffers."""
    from ferrl_b200.parallel.nvls import NvlsUnavailable
    try:
        red = GemmAllReducer(heap, 8192, 4096, nvls=True)
    except NvlsUnavailable as e:
        if rank == 0:
            print(f"TP_NVLS_UNAVAILABLE {e}")
        return
    failed = None
    try:
        _check_reducer(comm, heap, red, dev, world, rank, "in-switch fused all-reduce")
        t = _time(lambda: red(a, b, None, None, res))
        heap.check("in-switch timing")
        if rank == 0:
            print(f"TP_NVLS_TIMING world={world} M={a.shape[0]} N={b.shape[0]} K={a.shape[1]} fused_nvls_ms={t:.4f} gemm_nccl_ms={t_nccl:.4f}")
    except BaseException as e:  # noqa: BLE001
        failed = f"{type(e).__name__}: {e}"
    torch.cuda.synchronize()
    flags = comm.all_gather_bytes((failed or "").encode())
    assert not any(flags), [f.decode() for f in flags if f]
    if rank == 0:
        print("TP_NVLS_PASS")


def _sequence_parallel_checks(comm, heap, red, dev, world, rank):
    """Row collectives over the symmetric heap against the Comm seam, and a Gemma-style stack with the residual
    stream sharded over the token rows against the replicated layout (outputs and adapter gradients)."""
    from ferrl_b200.models.gemma4 import Gemma4GradModel, Gemma4Spec
    from ferrl_b200.models.lora import LoraSpec
    from ferrl_b200.parallel import sp
    from ferrl_b200.parallel.tp import TensorParallelPlan
    rc = sp.RowCollectives(heap, 4096 * 512 * 4)
    for it, (rows, cols, dtype) in enumerate([(64 * world, 512, torch.bfloat16), (3 * world, 37, torch.float32), (4096, 256, torch.bfloat16)]):
        gen = torch.Generator(device=dev).manual_seed(900 + 10 * it + rank)
        x = torch.randn(rows, cols, device=dev, generator=gen).to(dtype)
        got = rc.reduce_scatter(x)
        heap.check("reduce-scatter")
        want = sp._reduce_scatter_value(x, comm)                      # no collectives registered yet: Comm seam
        tol = (2.0 ** -7 if dtype == torch.bfloat16 else 1e-5) * max(1.0, float(want.float().abs().max()))
        assert got is not None and float((got.float() - want.float()).abs().max()) <= tol
        shard = got
        full = rc.all_gather(shard)
        heap.check("all-gather")
        assert full is not None and torch.equal(full, sp._all_gather_value(shard, comm))
    sp.register_row_collectives(comm, rc)
    hq = max(4, world)
    spec = Gemma4Spec(vocab_size=512 * world, hidden_size=256, num_hidden_layers=2, num_attention_heads=hq, num_key_value_heads=hq,
                      head_dim=64, global_head_dim=64, num_global_key_value_heads=hq, intermediate_size=512,
                      layer_types=["sliding_attention", "full_attention"], sliding_window=32, max_position_embeddings=128 * world)
    plan = TensorParallelPlan.new(rank, world, hq, hq, 512)
    # 128 x world token rows: whole tiles per rank, so the sharded layers run the fused GEMM -> reduce-scatter
    ids = torch.randint(0, spec.vocab_size, (2, 64 * world), device=dev, generator=torch.Generator(device=dev).manual_seed(5))
    outs = []
    fused_calls = [0]
    plain_rs = red.reduce_scatter

    def counted(*a, **k):
        fused_calls[0] += 1
        return plain_rs(*a, **k)
    red.reduce_scatter = counted
    for seq_par in (False, True):
        model = Gemma4GradModel(spec, LoraSpec(rank=8, alpha=16.0), dtype=torch.bfloat16, device=dev, tp=plan,
                                sequence_parallel=seq_par)
        model.init_random(seed=21)
        with torch.no_grad():
            for l in model.layers:          # scores are q.k without 1/sqrt(d): keep them of order ten, as trained norms do
                l.q_norm.fill_(0.3)
                l.k_norm.fill_(0.3)
            for i, q in enumerate(model.trainable_params()):
                q.copy_(torch.randn(q.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(70 + i)) * 0.05)
        h = model.forward_hidden(ids, comm)
        h.float().pow(2).mean().backward()
        outs.append((h.detach().float(), [q.grad.detach().float().clone() for q in model.trainable_params()]))
    heap.check("sequence-parallel model")
    red.reduce_scatter = plain_rs
    # per layer: o and down forward, qkv and gate_up backward (the first layer's qkv input, the frozen embedding, wants no gradient)
    assert fused_calls[0] >= 4 * spec.num_hidden_layers - 1, fused_calls[0]
    sp.register_row_collectives(comm, None)
    ref, got = outs
    assert float((ref[0] - got[0]).abs().max()) < 0.05 * float(ref[0].abs().max()), float((ref[0] - got[0]).abs().max())
    for g0, g1 in zip(ref[1], got[1]):
        assert float((g0 - g1).abs().max()) <= 0.08 * float(g0.abs().max()) + 1e-6
    comm.barrier()
    if rank == 0:
        print("TP_SEQUENCE_PARALLEL_PASS")


def main():
    comm = TorchDistComm.bootstrap(timeout_s=120.0)
    dev, world, rank = comm.device, comm.world_size, comm.rank
    heap = SymmHeap(comm, dev, wait_limit_s=20.0)
    red = GemmAllReducer(heap, 8192, 4096, gather_cols=256)    # gather buffers for the small sequence-sharded model below
    _check_reducer(comm, heap, red, dev, world, rank, "fused all-reduce")

    # timing: training-shaped row-parallel projection, fused vs. GEMM followed by NCCL
    M, N, K = 8192, 4096, 12288 // world
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) / K ** 0.5).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev).to(torch.bfloat16)
    t_fused = _time(lambda: red(a, b, None, None, res))

    def unfused():
        y = C.gemm(a, b)
        dist.all_reduce(y)
        return y + res
    t_nccl = _time(unfused)
    t_gemm = _time(lambda: C.gemm(a, b, None, None, res))
    heap.check("timing")
    _check_reduce_scatter(comm, heap, red, dev, world, rank)
    t_rs = _time(lambda: red.reduce_scatter(a, b))
    t_ar = _time(lambda: red(a, b))
    rs_out = torch.empty(M // world, N, device=dev, dtype=torch.bfloat16)

    def unfused_rs():
        dist.reduce_scatter_tensor(rs_out, C.gemm(a, b))
        return rs_out
    t_rs_nccl = _time(unfused_rs)
    heap.check("reduce-scatter timing")
    if rank == 0:
        print(f"TP_RS_TIMING world={world} M={M} N={N} K={K} fused_reduce_scatter_ms={t_rs:.4f} fused_all_reduce_ms={t_ar:.4f} "
              f"gemm_nccl_reduce_scatter_ms={t_rs_nccl:.4f}")
    if rank == 0:
        print(f"TP_TIMING world={world} M={M} N={N} K={K} fused_ms={t_fused:.4f} gemm_nccl_ms={t_nccl:.4f} "
              f"gemm_only_ms={t_gemm:.4f}")
    if os.environ.get("FERRL_TEST_NVLS") == "1":
        _nvls_variant(comm, heap, dev, world, rank, a, b, res, t_nccl)

    # model-level equivalence: tensor-parallel layers with and without the fused kernel
    from ferrl_b200.models.dense import DenseGradModel, DenseSpec
    from ferrl_b200.models.lora import LoraSpec
    from ferrl_b200.parallel.tp import TensorParallelPlan
    hq, hkv = max(4, world), max(2, world)          # heads divide evenly over 2, 4 and 8 ranks
    spec = DenseSpec(vocab_size=512, hidden_size=256, num_hidden_layers=2, num_attention_heads=hq,
                     num_key_value_heads=hkv, head_dim=64, intermediate_size=512)
    plan = TensorParallelPlan.new(rank, world, hq, hkv, 512)
    ids = torch.randint(0, spec.vocab_size, (2, 64), device=dev, generator=torch.Generator(device=dev).manual_seed(3))
    outs = []
    for fused_on in (False, True):
        model = DenseGradModel(spec, LoraSpec(rank=8, alpha=16.0), dtype=torch.bfloat16, device=dev, tp=plan)
        model.init_random(seed=11)
        with torch.no_grad():   # non-zero B so that both adapter factors get a gradient
            for i, q in enumerate(model.trainable_params()):
                q.copy_(torch.randn(q.shape, device=dev, generator=torch.Generator(device=dev).manual_seed(50 + i)) * 0.05)
        if fused_on:
            register_gemm_all_reducer(comm, red)
        logits = model(ids, comm)
        logits.pow(2).mean().backward()
        outs.append((logits.detach(), [q.grad.detach().float().clone() for q in model.trainable_params()]))
    heap.check("tensor-parallel model")
    assert float((outs[0][0] - outs[1][0]).abs().max()) < 0.05 * float(outs[0][0].abs().max())
    for g0, g1 in zip(outs[0][1], outs[1][1]):
        assert float((g0 - g1).abs().max()) <= 0.08 * float(g0.abs().max()) + 1e-6
    # vocabulary-sharded log-prob head: each rank scores 1 / world of the vocabulary in the head GEMM's epilogue
    from ferrl_b200.parallel.tp import sharded_logprob_gather
    gen = torch.Generator(device=dev).manual_seed(23)
    Nr, Hh, Vv = 700, 256, 1024 * world
    hh = (torch.randn(Nr, Hh, device=dev, generator=gen) * 0.7).to(torch.bfloat16)
    ww = (torch.randn(Vv, Hh, device=dev, generator=gen) * 0.05).to(torch.bfloat16)
    tt = torch.randint(0, Vv, (Nr,), device=dev, generator=gen)
    dlp = torch.randn(Nr, device=dev, generator=gen)
    for cap, temp in ((0.0, 1.0), (30.0, 0.7)):
        h1 = hh.clone().requires_grad_()
        lp1 = sharded_logprob_gather(h1, ww, tt, temp, cap, comm)
        assert lp1 is not None
        lp1.backward(dlp)
        h2 = hh.clone().requires_grad_()
        lp2 = C.logprob_gather(h2, ww, tt, temp, cap)
        lp2.backward(dlp)
        heap.check("sharded head")
        assert float((lp1 - lp2).abs().max()) < 2e-3 * max(1.0, float(lp2.abs().max())), float((lp1 - lp2).abs().max())
        rel = float((h1.grad.float() - h2.grad.float()).norm() / h2.grad.float().norm())
        assert rel < 1.5e-2, rel
        comm.require_consensus(hashlib.sha256(lp1.detach().cpu().numpy().tobytes()).digest(), "sharded head log-probs")
    comm.barrier()
    if rank == 0:
        print("TP_SHARDED_HEAD_PASS")
    _sequence_parallel_checks(comm, heap, red, dev, world, rank)
    _check_gather_gemm(comm, heap, dev, world, rank)
    if rank == 0:
        print("TP_FUSED_PASS")
    dist.destroy_process_group()


if __name__ == "__main__":
    sys.exit(main())
