"""Fused data-parallel step: single-GPU emulation of several ranks' data (one launch, no
cross-launch waiting), and the real multi-process path when at least two GPUs are visible."""
import math
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _need_gpu(n=1):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} CUDA device(s)")


@pytest.mark.parametrize("max_norm", [None, 0.5])
def test_fused_step_emulated_world4_matches_eager(max_norm):
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import eager as E
    from ferrl_b200.optim import AdamWParams, FerrlAdamW
    from ferrl_b200.parallel.dp import FusedDpStep
    from ferrl_b200.parallel.symm import SymmHeap
    dev = torch.device("cuda", 0)
    torch.manual_seed(0)
    shapes = [(16, 512), (512, 16), (7, 3), (40000,)]
    params = [torch.nn.Parameter(torch.randn(s, device=dev)) for s in shapes]
    ref_p = [p.detach().clone() for p in params]
    opt = FerrlAdamW(params, AdamWParams(lr=1e-2, weight_decay=0.01))
    ref_m, ref_v = [torch.zeros_like(p) for p in ref_p], [torch.zeros_like(p) for p in ref_p]
    fused = FusedDpStep(SymmHeap(SoloComm(), dev), params, emulate_world=4)
    for step in range(1, 4):
        fused.prepare_grads()
        gs = [torch.randn(s, device=dev) for s in shapes]
        for p, g in zip(params, gs):
            p.grad.add_(g)
            p.grad = p.grad  # keep the view
        res = fused(opt, None, max_norm, 0.0, pre_scale=0.25)
        red = [g * 4 * 0.25 for g in gs]           # four identical "ranks", scaled by 1/world
        norm = math.sqrt(sum(float(g.double().pow(2).sum()) for g in red))
        assert res.stepped and abs(res.grad_norm - norm) / norm < 1e-5
        scale = 1.0 if max_norm is None or norm <= max_norm else max_norm / norm
        E.adamw_step(ref_p, red, ref_m, ref_v, lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01,
                     step=step, grad_scale=scale)
        for a, b in zip(params, ref_p):
            assert (a.detach() - b).abs().max().item() < 2e-5
    assert opt.step_t == 3
    # non-finite gradient anywhere => nobody steps
    fused.prepare_grads()
    params[0].grad[0, 0] = float("nan")
    before = [p.detach().clone() for p in params]
    res = fused(opt, None, max_norm, 0.0)
    assert not res.stepped and res.uncovered > 0 and opt.step_t == 3
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, params))
    # all-zero gradient => skip
    fused.prepare_grads()
    res = fused(opt, None, max_norm, 0.0)
    assert not res.stepped and res.grad_norm == 0.0


def test_symm_all_reduce_world1():
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.parallel.symm import SymmAllReducer, SymmHeap
    dev = torch.device("cuda", 0)
    red = SymmAllReducer(SymmHeap(SoloComm(), dev), 1 << 20)
    x = torch.randn(33, 128, device=dev).to(torch.bfloat16)
    assert torch.equal(red(x), x)


def test_peer_wait_times_out_without_hanging():
    """A barrier that nobody else joins must run out, report through the status word and leave
    the context usable (the wait is bounded to a fraction of a second here)."""
    _need_gpu()
    from ferrl_b200.comm import CommTimeout, SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.symm import SymmBuffer, SymmHeap
    dev = torch.device("cuda", 0)
    heap = SymmHeap(SoloComm(), dev, wait_limit_s=0.3)
    buf = heap.alloc(4096)
    out = torch.zeros(1024, dtype=torch.float32, device=dev)
    # pretend there is a second rank whose flag slot is never written
    fake = SymmBuffer(buf.local, [buf.ptrs[0], buf.ptrs[0]])
    C.lib().symm_all_reduce(fake.ptrs, [heap.flags.ptrs[0]] * 2, out, 0, 2, heap.next_epoch() + 5, 0.3, heap.abort_word)
    with pytest.raises(CommTimeout):
        heap.check("test all-reduce")
    assert C.kernel_status() == 0
    y = torch.ones(8, device=dev) * 2           # context still works
    assert float(y.sum()) == 16.0


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_process_dp_step_and_all_reduce(world):
    _need_gpu(world)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29650 + world), os.path.join(ROOT, "tests", "multi_gpu_dp_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "DP_STEP_PASS" in res.stdout
