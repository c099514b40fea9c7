"""Fused row-parallel GEMM -> all-reduce kernel.

On one GPU the peer is played by the host: its partial tiles, ready flags, reduced tiles and done
flags are written before the launch, so the kernel under test never waits on another launch.  The
check covers every byte the kernel must produce: its own output, the partial tiles and flags it
pushes to the peer, and the reduced tiles it sends back.  The real two-process run lives in
``multi_gpu_tp_worker.py``.
"""
import os
import subprocess
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
BM, MAXR = 128, 16


def _need_gpu(n=1):
    if not torch.cuda.is_available() or torch.cuda.device_count() < n:
        pytest.skip(f"needs {n} CUDA device(s)")


def _chunk_major(tile):
    """[128, BN] row-major tile -> staging layout [BN/8][128][8]."""
    return tile.reshape(BM, -1, 8).permute(1, 0, 2).reshape(-1)


def _tiles(M, N, BN):
    return (M + BM - 1) // BM, (N + BN - 1) // BN


def _pad_tile(full, mi, ni, BN):
    t = torch.zeros(BM, BN, dtype=full.dtype, device=full.device)
    src = full[mi * BM:(mi + 1) * BM, ni * BN:(ni + 1) * BN]
    t[:src.shape[0], :src.shape[1]] = src
    return t


@pytest.mark.parametrize("M,N,K,rank,res,lora", [(300, 512, 256, 0, False, False), (300, 512, 256, 1, True, True),
                                                  (128, 4096, 2048, 0, True, False)])
def test_rank_against_host_played_peer(M, N, K, rank, res, lora):
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.symm import GemmAllReducer, SymmHeap
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M + N + K + rank)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    peer = 1 - rank
    a = [rnd(M, K).to(torch.bfloat16) for _ in range(2)]
    b = [(rnd(N, K) / K ** 0.5).to(torch.bfloat16) for _ in range(2)]
    t2 = [rnd(M, 16).to(torch.bfloat16) for _ in range(2)] if lora else [None, None]
    b2 = (rnd(N, 16) * 0.1).to(torch.bfloat16) if lora else None
    residual = rnd(M, N).to(torch.bfloat16) if res else None
    part = []
    for r in range(2):
        p = a[r].float() @ b[r].float().t()
        if lora:
            p = p + t2[r].float() @ b2.float().t()
        part.append(p.to(torch.bfloat16))
    total = part[0].float() + part[1].float()
    if res:
        total = total + residual.float()
    want = total.to(torch.bfloat16)

    heap = SymmHeap(SoloComm(), dev, wait_limit_s=0.5)
    red = GemmAllReducer(heap, M, N)
    BN = 128                                   # the binding picks 128 for these (small) problems
    mt, nt = _tiles(M, N, BN)
    slot = BM * BN
    mine = dict(stage=red.stage.local.view(torch.bfloat16), out=red.outbuf.local.view(torch.bfloat16),
                flags=red.flags.local.view(torch.int32))
    theirs = dict(stage=torch.zeros_like(mine["stage"]), out=torch.zeros_like(mine["out"]),
                  flags=torch.zeros_like(mine["flags"]))
    epoch = 7
    done_base = red.max_tiles * MAXR
    mine["flags"][red.max_tiles * (MAXR + 1)] = epoch - 1      # device-resident call counter: this call is number 7
    fin_base = red.max_tiles * (MAXR + 1) + 2
    mine["flags"][fin_base + peer] = epoch - 1                  # the peer has left the previous call
    for t in range(mt * nt):
        mi, ni = divmod(t, nt)
        if t % 2 == rank:     # mine to reduce: the peer's partial is already in my staging slot
            off = ((t // 2) * 2 + peer) * slot
            mine["stage"][off:off + slot] = _chunk_major(_pad_tile(part[peer], mi, ni, BN))
            mine["flags"][t * MAXR + peer] = epoch
        else:                 # the peer's to reduce: its result is already in my output buffer
            rows = slice(mi * BM, min(M, (mi + 1) * BM))
            cols = slice(ni * BN, min(N, (ni + 1) * BN))
            mine["out"][:M * N].view(M, N)[rows, cols] = want[rows, cols]
            mine["flags"][done_base + t] = epoch
    ptrs = lambda key: [(mine if r == rank else theirs)[key].data_ptr() for r in range(2)]
    torch.cuda.synchronize()
    y = C.lib().gemm_allreduce(a[rank], b[rank], t2[rank], b2, residual, ptrs("stage"), ptrs("out"), ptrs("flags"),
                               rank, 2, epoch, red.max_tiles, red.stage_elems, red.out_elems, 0.5)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    assert int(mine["flags"][red.max_tiles * (MAXR + 1)]) == epoch      # the kernel advanced its own counter
    assert int(theirs["flags"][fin_base + rank]) == epoch               # and told the peer that it has left this call
    tol = 0.02 * float(want.float().abs().max())
    assert float((y.float() - want.float()).abs().max()) <= tol
    peer_out = theirs["out"][:M * N].view(M, N)
    for t in range(mt * nt):
        mi, ni = divmod(t, nt)
        rows = slice(mi * BM, min(M, (mi + 1) * BM))
        cols = slice(ni * BN, min(N, (ni + 1) * BN))
        if t % 2 == rank:
            # reduced tile delivered to the peer, bit-identical to my own copy, and announced
            assert torch.equal(peer_out[rows, cols], y[rows, cols])
            assert int(theirs["flags"][done_base + t]) == epoch
        else:
            off = ((t // 2) * 2 + rank) * slot
            got = theirs["stage"][off:off + slot].reshape(BN // 8, BM, 8).permute(1, 0, 2).reshape(BM, BN)
            ref = _pad_tile(part[rank], mi, ni, BN)
            assert float((got.float() - ref.float()).abs().max()) <= tol
            assert int(theirs["flags"][t * MAXR + rank]) == epoch
            assert torch.equal(y[rows, cols], want[rows, cols])     # copied verbatim from my output buffer


@pytest.mark.parametrize("rank,lora", [(0, False), (1, True)])
def test_reduce_scatter_form_against_host_played_peer(rank, lora):
    """Reduce-scatter form: this rank keeps its own row block of the sum, pushes its partials of the peer's block
    and sends nothing back."""
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.symm import GemmAllReducer, SymmHeap
    dev = torch.device("cuda", 0)
    M, N, K, BN = 512, 512, 256, 128
    g = torch.Generator(device=dev).manual_seed(91 + rank)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    peer = 1 - rank
    a = [rnd(M, K).to(torch.bfloat16) for _ in range(2)]
    b = [(rnd(N, K) / K ** 0.5).to(torch.bfloat16) for _ in range(2)]
    t2 = [rnd(M, 16).to(torch.bfloat16) for _ in range(2)] if lora else [None, None]
    b2 = (rnd(N, 16) * 0.1).to(torch.bfloat16) if lora else None
    part = []
    for r in range(2):
        p = a[r].float() @ b[r].float().t()
        if lora:
            p = p + t2[r].float() @ b2.float().t()
        part.append(p.to(torch.bfloat16))
    want = (part[0].float() + part[1].float()).to(torch.bfloat16)
    heap = SymmHeap(SoloComm(), dev, wait_limit_s=0.5)
    red = GemmAllReducer(heap, M, N)
    mt, nt = _tiles(M, N, BN)
    mt_per, slot = mt // 2, BM * BN
    mine = dict(stage=red.stage.local.view(torch.bfloat16), flags=red.flags.local.view(torch.int32))
    theirs = dict(stage=torch.zeros_like(mine["stage"]), flags=torch.zeros_like(mine["flags"]))
    spare_out = torch.zeros_like(red.outbuf.local)
    epoch = 5
    ctr = red.max_tiles * (MAXR + 1)
    mine["flags"][ctr] = epoch - 1
    mine["flags"][ctr + 2 + peer] = epoch - 1
    local_slot = lambda mi, ni, owner, frm: (((mi - owner * mt_per) * nt + ni) * 2 + frm) * slot
    for mi in range(rank * mt_per, (rank + 1) * mt_per):          # my row block: the peer's partials are already here
        for ni in range(nt):
            off = local_slot(mi, ni, rank, peer)
            mine["stage"][off:off + slot] = _chunk_major(_pad_tile(part[peer], mi, ni, BN))
            mine["flags"][(mi * nt + ni) * MAXR + peer] = epoch
    ptrs = lambda key: [(mine if r == rank else theirs)[key].data_ptr() for r in range(2)]
    outs = [red.outbuf.local.data_ptr() if r == rank else spare_out.data_ptr() for r in range(2)]
    torch.cuda.synchronize()
    y = C.lib().gemm_allreduce(a[rank], b[rank], t2[rank], b2, None, ptrs("stage"), outs, ptrs("flags"), rank, 2, epoch,
                               red.max_tiles, red.stage_elems, red.out_elems, 0.5, None, 0, 0, True)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    n = M // 2
    tol = 0.02 * float(want.float().abs().max())
    assert y.shape == (n, N)
    assert float((y.float() - want[rank * n:(rank + 1) * n].float()).abs().max()) <= tol
    for mi in range(peer * mt_per, (peer + 1) * mt_per):          # the peer's row block: my partials and their flags
        for ni in range(nt):
            off = local_slot(mi, ni, peer, rank)
            got = theirs["stage"][off:off + slot].reshape(BN // 8, BM, 8).permute(1, 0, 2).reshape(BM, BN)
            assert float((got.float() - _pad_tile(part[rank], mi, ni, BN).float()).abs().max()) <= tol
            assert int(theirs["flags"][(mi * nt + ni) * MAXR + rank]) == epoch
    assert int(mine["flags"][ctr]) == epoch and int(theirs["flags"][ctr + 2 + rank]) == epoch
    assert not bool(spare_out.any())                               # nothing is sent back in this form


@pytest.mark.parametrize("rank,K", [(0, 256), (1, 264)])
def test_all_gather_form_against_host_played_peer(rank, K):
    """All-gather form: the peer's rows sit in its buffer (here: a second local buffer) with its "rows in place" flag
    set; the kernel pulls them into this rank's buffer and multiplies all rows."""
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.symm import GemmAllReducer, SymmHeap
    dev = torch.device("cuda", 0)
    M, N = 512, 384
    g = torch.Generator(device=dev).manual_seed(17 + rank)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(N, K, device=dev, generator=g) / K ** 0.5).to(torch.bfloat16)
    peer, n = 1 - rank, M // 2
    heap = SymmHeap(SoloComm(), dev, wait_limit_s=0.5)
    red = GemmAllReducer(heap, M, N, gather_cols=K)
    mine_buf = red.gather_bufs[0].local[:M * K * 2].view(torch.bfloat16).view(M, K)
    mine_buf.zero_()
    mine_buf[rank * n:(rank + 1) * n] = x[rank * n:(rank + 1) * n]
    their_buf = torch.zeros(M, K, device=dev, dtype=torch.bfloat16)
    their_buf[peer * n:(peer + 1) * n] = x[peer * n:(peer + 1) * n]
    flags = red.flags.local.view(torch.int32)
    their_flags = torch.zeros_like(flags)
    epoch = 9
    ctr = red.max_tiles * (MAXR + 1)
    agr, arrived = ctr + 2 + MAXR, ctr + 2 + 2 * MAXR
    flags[ctr] = epoch - 1
    flags[agr + peer] = epoch                                      # the peer's rows are in place
    bufs = [mine_buf.data_ptr() if r == rank else their_buf.data_ptr() for r in range(2)]
    fl = [flags.data_ptr() if r == rank else their_flags.data_ptr() for r in range(2)]
    torch.cuda.synchronize()
    y = C.lib().gemm_allgather(w, None, None, bufs, fl, rank, 2, red.max_tiles, M, K, 0.5)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    assert torch.equal(mine_buf, x)
    ref = x.float() @ w.float().t()
    assert float((y.float() - ref).abs().max()) <= 0.02 * float(ref.abs().max())
    assert int(flags[ctr]) == epoch and int(their_flags[agr + rank]) == epoch
    assert not bool(flags[arrived:arrived + M // BM].any())         # arrival counts are back to zero for the next call


def test_missing_peer_runs_out_without_hanging():
    """No peer ever signals: the owner's wait must expire, the status word must say so and the
    context must stay usable."""
    _need_gpu()
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.symm import GemmAllReducer, SymmHeap
    dev = torch.device("cuda", 0)
    heap = SymmHeap(SoloComm(), dev, wait_limit_s=0.3)
    red = GemmAllReducer(heap, 256, 256)
    a = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    b = torch.randn(256, 128, device=dev).to(torch.bfloat16)
    spare = {k: torch.zeros_like(getattr(red, k).local) for k in ("stage", "outbuf", "flags")}
    ptrs = lambda k: [getattr(red, k).local.data_ptr(), spare[k].data_ptr()]
    C.lib().gemm_allreduce(a, b, None, None, None, ptrs("stage"), ptrs("outbuf"), ptrs("flags"), 0, 2, 3,
                           red.max_tiles, red.stage_elems, red.out_elems, 0.3)
    torch.cuda.synchronize()
    assert C.kernel_status() != 0
    C.lib().reset_status()
    y = C.gemm(a, b)                              # the same kernel family still runs
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    assert float((y.float() - a.float() @ b.float().t()).abs().max()) < 1.0


def _torchrun(worker, world, port, marker, timeout=900):
    """One rank per GPU; NVLS off: a rank that fails between kernels must not leave multicast bindings behind."""
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(port), os.path.join(ROOT, "tests", worker)]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=timeout)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert marker in res.stdout
    return res.stdout


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_process_fused_tp(world):
    _need_gpu(world)
    out = _torchrun("multi_gpu_tp_worker.py", world, 29613 + world, "TP_FUSED_PASS")
    print("\n".join(l for l in out.splitlines() if l.startswith("TP_")))
    if os.environ.get("FERRL_TEST_NVLS") == "1":          # the in-switch variant ran too, or said why it could not
        assert "TP_NVLS_PASS" in out or "TP_NVLS_UNAVAILABLE" in out


@pytest.mark.parametrize("world", [2, 4, 8])
def test_multi_process_expert_parallel(world):
    _need_gpu(world)
    out = _torchrun("multi_gpu_ep_worker.py", world, 29633 + world, "EP_PASS")
    print("\n".join(l for l in out.splitlines() if l.startswith("EP_")))
    assert "EP_GRAPH_REPLAY_PASS" in out


@pytest.mark.parametrize("world", [int(w) for w in os.environ.get("FERRL_TEST_NVLS_WORLDS", "2").split(",")])
def test_multi_process_nvls_all_reduce(world):
    """In-switch all-reduce (multimem) against the peer-load form; passes with a note where the box has no multicast.
    World size 2 by default; ``FERRL_TEST_NVLS_WORLDS=2,4,8`` runs the larger groups too."""
    _need_gpu(world)
    env = dict(os.environ, NCCL_NVLS_ENABLE="0", PYTHONPATH=ROOT)
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr",
           "127.0.0.1", "--master-port", str(29653 + world), os.path.join(ROOT, "tests", "multi_gpu_nvls_worker.py")]
    res = subprocess.run(cmd, env=env, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "NVLS_PASS" in res.stdout or "NVLS_UNAVAILABLE" in res.stdout
    print("\n".join(l for l in res.stdout.splitlines() if l.startswith("NVLS_")))
