"""Two-SM (cta_group::2) GEMM against fp32 matmul."""
import pytest
import torch

from _numerics import close as _close   # norm ratio AND an elementwise bound

pytestmark = pytest.mark.gpu

WIDTHS = (128, 256)


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("bn", WIDTHS)
@pytest.mark.parametrize("M,N,K,res,lora", [(256, 256, 64, False, False), (512, 512, 256, True, False),
                                             (1000, 384, 520, False, True), (4096, 4096, 1024, True, True),
                                             (300, 136, 72, True, False)])
def test_two_cta_matches_fp32(bn, M, N, K, res, lora):
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    a = rnd(M, K).to(torch.bfloat16)
    b = (rnd(N, K) / K ** 0.5).to(torch.bfloat16)
    a2 = rnd(M, 16).to(torch.bfloat16) if lora else None
    b2 = (rnd(N, 16) * 0.2).to(torch.bfloat16) if lora else None
    r = rnd(M, N).to(torch.bfloat16) if res else None
    dbg = torch.zeros(2, dtype=torch.int32, device=dev)
    y = C.gemm(a, b, a2, b2, r, two_cta=bn, debug=dbg)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    want = a.float() @ b.float().t()
    if lora:
        want = want + a2.float() @ b2.float().t()
    if res:
        want = want + r.float()
    print("tmem bases of the CTA pair:", dbg.tolist())
    assert dbg[0].item() == dbg[1].item()
    err = float((y.float() - want).abs().max())
    assert err <= 0.02 * float(want.abs().max()), err
    # same bits as the one-SM kernel (same k order, same rounding)
    y1 = C.gemm(a, b, a2, b2, r, force_bn=128 if N >= 128 else 64)
    assert float((y.float() - y1.float()).abs().max()) <= 0.01 * float(want.abs().max())


@pytest.mark.parametrize("bn,S", [(64, 2), (64, 4), (128, 2), (128, 4), (128, 8), (256, 2)])
@pytest.mark.parametrize("M,N,K,res,lora,f32", [(128, 512, 4096, False, False, False), (100, 1024, 1032, True, True, False),
                                                 (256, 768, 192, True, False, True), (7, 256, 64, False, False, False)])
def test_cluster_split_k(bn, S, M, N, K, res, lora, f32):
    """Cluster split-k (partials reduced through distributed shared memory) against fp32 matmul,
    including k-slices that come out empty and repeated calls (bitwise reproducible)."""
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(M + N + K + bn + S)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    a = rnd(M, K).to(torch.bfloat16)
    b = (rnd(N, K) / K ** 0.5).to(torch.bfloat16)
    a2 = rnd(M, 16).to(torch.bfloat16) if lora else None
    b2 = (rnd(N, 16) * 0.2).to(torch.bfloat16) if lora else None
    r = rnd(M, N).to(torch.bfloat16) if res else None
    y = C.gemm(a, b, a2, b2, r, out_f32=f32, force_bn=bn, cluster_k=S)
    y2 = C.gemm(a, b, a2, b2, r, out_f32=f32, force_bn=bn, cluster_k=S)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    want = a.float() @ b.float().t()
    if lora:
        want = want + a2.float() @ b2.float().t()
    if res:
        want = want + r.float()
    assert float((y.float() - want).abs().max()) <= 0.02 * float(want.abs().max())
    assert torch.equal(y, y2)


@pytest.mark.parametrize("M,N,K", [(128, 6144, 4096), (128, 4096, 4096), (128, 24576, 4096), (128, 4096, 12288),
                                   (128, 151936, 4096), (200, 4096, 4096)])
def test_decode_shapes_planned(M, N, K):
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(N + K)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev, generator=g) / K ** 0.5).to(torch.bfloat16)
    y = C.gemm(a, b)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    want = a.float() @ b.float().t()
    assert float((y.float() - want).abs().max()) <= 0.02 * float(want.abs().max())


@pytest.mark.parametrize("M,N,K,res,lora,f32", [(128, 6144, 4096, False, False, False), (128, 4096, 4096, True, False, False),
                                                 (128, 24576, 4096, False, False, False), (100, 4096, 12288, True, True, False),
                                                 (128, 151936, 4096, False, False, True), (7, 1000, 520, True, True, False),
                                                 (128, 256, 64, False, False, False)])
def test_stream_k(M, N, K, res, lora, f32):
    """Stream-k decode GEMM (equal unit ranges per SM, partial tiles fixed up through L2) against
    fp32 matmul; repeated launches must agree bit for bit (fixed summation order, self-advancing
    launch counter)."""
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    a = rnd(M, K).to(torch.bfloat16)
    b = (rnd(N, K) / K ** 0.5).to(torch.bfloat16)
    a2 = rnd(M, 16).to(torch.bfloat16) if lora else None
    b2 = (rnd(N, 16) * 0.2).to(torch.bfloat16) if lora else None
    r = rnd(M, N).to(torch.bfloat16) if res else None
    ys = [C.gemm(a, b, a2, b2, r, out_f32=f32, stream_k=1) for _ in range(3)]
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    want = a.float() @ b.float().t()
    if lora:
        want = want + a2.float() @ b2.float().t()
    if res:
        want = want + r.float()
    assert float((ys[0].float() - want).abs().max()) <= 0.02 * float(want.abs().max())
    assert torch.equal(ys[0], ys[1]) and torch.equal(ys[1], ys[2])
    # replay inside a CUDA graph: the launch counter lives on the device
    graph = torch.cuda.CUDAGraph()
    static = torch.empty_like(ys[0])
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        static.copy_(C.gemm(a, b, a2, b2, r, out_f32=f32, stream_k=1))
    torch.cuda.current_stream().wait_stream(s)
    with torch.cuda.graph(graph):
        static.copy_(C.gemm(a, b, a2, b2, r, out_f32=f32, stream_k=1))
    for _ in range(3):
        static.zero_()
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(static, ys[0])
    assert C.kernel_status() == 0


@pytest.mark.parametrize("M,N,K", [(128, 6144, 4096), (128, 4096, 12288), (64, 24576, 4096), (7, 512, 192)])
def test_gemm_dependent_launch_orders_activations(M, N, K):
    """`static_b=True` launches a decode-shaped GEMM as a programmatic dependent: its weight tiles
    stream while the previous kernel runs, the activation tiles only after it has finished.  The
    activations are rewritten by the kernel just before every call, eagerly and in a replayed graph."""
    from ferrl_b200.ops import cuda as C
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M + N)
    w = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    a = torch.empty_like(x)

    def step(scale):
        torch.mul(x, scale, out=a)                 # the predecessor writes the activations
        y = C.gemm(a, w, static_b=True)
        return y

    for i in range(6):
        sc = 1.0 + 0.25 * i
        y = step(sc)
        ref = (x.float() * sc).to(torch.bfloat16).float() @ w.float().t()
        _close(y, ref, 1e-2)
    assert C.kernel_status() == 0
    sc_t = torch.ones((), device=dev)
    torch.cuda.synchronize()
    gr = torch.cuda.CUDAGraph()
    with torch.cuda.graph(gr):
        torch.mul(x, sc_t, out=a)
        yg = C.gemm(a, w, static_b=True)
        yg2 = C.gemm(yg[:, :K].contiguous() if N >= K else a, w, static_b=True)   # GEMM after GEMM-fed kernel
    for i in range(4):
        sc_t.fill_(0.5 + i)
        gr.replay()
        torch.cuda.synchronize()
        ref = (x.float() * (0.5 + i)).to(torch.bfloat16).float() @ w.float().t()
        _close(yg, ref, 1e-2)
    assert C.kernel_status() == 0


def test_dependent_launch_chain_matches_reference():
    """A decode-layer-like chain (RMSNorm -> projection -> GLU -> projection with residual) in which
    every kernel is a programmatic dependent of the one before it, replayed from a CUDA graph with
    fresh inputs, against the same chain in fp32."""
    from ferrl_b200.ops import cuda as C
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    Bt, H, F = 128, 1024, 2048
    x = torch.randn(Bt, H, device=dev, generator=g).to(torch.bfloat16)
    wn = (1 + 0.1 * torch.randn(H, device=dev, generator=g)).to(torch.bfloat16)
    w1 = (torch.randn(2 * F, H, device=dev, generator=g) * 0.03).to(torch.bfloat16)
    w2 = (torch.randn(H, F, device=dev, generator=g) * 0.03).to(torch.bfloat16)

    def chain(inp):
        h = C.rmsnorm(inp, wn, 1e-6)
        gu = C.gemm(h, w1, static_b=True)
        a = C.swiglu(gu)
        return C.gemm(a, w2, residual=inp, static_b=True)

    def ref(inp):
        xf = inp.float()
        h = (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + 1e-6) * wn.float()).to(torch.bfloat16).float()
        gu = (h @ w1.float().t()).to(torch.bfloat16).float()
        a = (torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]).to(torch.bfloat16).float()
        return xf + a @ w2.float().t()

    with torch.no_grad():
        y = chain(x)
        r = ref(x)
        _close(y, r, 2e-2)
        xin = x.clone()
        torch.cuda.synchronize()
        gr = torch.cuda.CUDAGraph()
        with torch.cuda.graph(gr):
            yg = chain(xin)
        for i in range(5):
            xin.copy_(torch.randn(Bt, H, device=dev, generator=g).to(torch.bfloat16))
            gr.replay()
            torch.cuda.synchronize()
            r = ref(xin)
            _close(yg, r, 2e-2)
    assert C.kernel_status() == 0


@pytest.mark.parametrize("M,F,K,act", [(128, 12288, 4096, "silu"), (7, 88, 192, "silu"), (300, 1024, 512, "gelu_tanh"),
                                         (2048, 2048, 1024, "silu")])
def test_gemm_glu_epilogue(M, F, K, act):
    """Projection with the GLU in its epilogue (gate/up rows interleaved in groups of 16) against
    act(x Wg^T) * (x Wu^T) in fp32."""
    from ferrl_b200.ops import cuda as C
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(F + M)
    x = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(2 * F, K, device=dev, generator=g) * (2.0 / K ** 0.5)).to(torch.bfloat16)
    idx = torch.arange(F, device=dev).view(-1, 8)
    perm = torch.stack([idx, idx + F], dim=1).reshape(-1)
    y = C.gemm_glu(x, w.index_select(0, perm).contiguous(), act)
    gu = x.float() @ w.float().t()
    gate, up = gu[:, :F], gu[:, F:]
    a = torch.nn.functional.silu(gate) if act == "silu" else torch.nn.functional.gelu(gate, approximate="tanh")
    ref = a * up
    assert y.shape == (M, F)
    _close(y, ref, 1e-2)
    assert C.kernel_status() == 0


def test_fused_linear_glu_layout_matches_plain_snapshot():
    """A gate/up projection whose merged snapshot is kept interleaved gives the same rollout
    activations as projection + GLU kernel on the plain snapshot, and still serves plain calls."""
    from ferrl_b200.models.lora import FusedLoraLinear, LoraSpec
    from ferrl_b200 import ops
    dev = torch.device("cuda", 0)
    torch.manual_seed(3)
    H, F = 512, 1024
    mk = lambda: FusedLoraLinear(H, [F, F], ("gate", "up"), (True, True), LoraSpec(rank=8, alpha=16.0),  # noqa: E731
                                 dtype=torch.bfloat16, device=dev)
    a, b = mk(), mk()
    w = (torch.randn(2 * F, H, device=dev) * 0.05).to(torch.bfloat16)
    for m in (a, b):
        m.set_weight(w)
    for pa, pb in zip(list(a.lora_A) + list(a.lora_B), list(b.lora_A) + list(b.lora_B)):
        v = torch.randn_like(pa) * 0.05
        pa.data.copy_(v)
        pb.data.copy_(v)
    b.enable_glu_layout()
    a.merge()
    b.merge()
    x = torch.randn(64, H, device=dev).to(torch.bfloat16)
    with torch.no_grad():
        ref = ops.swiglu(a.forward_merged(x), "silu")
        got = b.forward_merged_glu(x, "silu")
        plain = b.forward_merged(x)
    _close(got, ref, 1e-2)
    assert torch.equal(plain, a.forward_merged(x))


@pytest.mark.parametrize("M,N,K", [(128, 6144, 4096), (128, 4096, 12288), (96, 4096, 4096), (128, 1024, 512), (300, 2048, 1024)])
def test_gemm_folded_rmsnorm_chain(M, N, K):
    """RMSNorm folded around projections: the producer's epilogue writes partial row sums of squares of
    what it stores, the consumer scales its rows by the resulting rstd and reads weights that carry
    the norm weight, against rmsnorm + matmul in fp32."""
    from ferrl_b200.ops import cuda as C
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M + N + K)
    eps = 1e-6
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    w1 = (torch.randn(N, K, device=dev, generator=g) / K ** 0.5).to(torch.bfloat16)
    res = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16)
    # producer: h = res + a w1^T, with row statistics
    h, ss = C.gemm_norm(a, w1, res, None, 0.0, None, True)
    h_ref = res.float() + a.float() @ w1.float().t()
    _close(h, h_ref, 1e-2)
    assert ss.dim() == 2 and ss.shape[1] == M
    ss_ref = h.float().pow(2).sum(-1)
    assert ((ss.sum(0) - ss_ref).abs() / ss_ref).max().item() < 1e-4
    assert torch.equal(ss, C.gemm_norm(a, w1, res, None, 0.0, None, True)[1])       # fixed order
    # consumer: y = rmsnorm(h, wn) w2^T through the folded weight
    wn = (1 + 0.2 * torch.randn(N, device=dev, generator=g)).to(torch.bfloat16)
    w2 = (torch.randn(512, N, device=dev, generator=g) / N ** 0.5).to(torch.bfloat16)
    folded = (w2.float() * wn.float()[None, :]).to(torch.bfloat16)
    y, none = C.gemm_norm(h, folded, None, ss, eps)
    assert none is None
    hf = h.float()
    xn = hf * torch.rsqrt(hf.pow(2).mean(-1, keepdim=True) + eps) * wn.float()
    y_ref = xn @ w2.float().t()
    _close(y, y_ref, 1.5e-2)
    # consumer with the GLU epilogue
    F = 256
    wg = (torch.randn(2 * F, N, device=dev, generator=g) / N ** 0.5).to(torch.bfloat16)
    idx = torch.arange(F, device=dev).view(-1, 8)
    perm = torch.stack([idx, idx + F], dim=1).reshape(-1)
    wgf = (wg.float() * wn.float()[None, :]).to(torch.bfloat16).index_select(0, perm).contiguous()
    z, _ = C.gemm_norm(h, wgf, None, ss, eps, "silu")
    gu = xn @ wg.float().t()
    z_ref = torch.nn.functional.silu(gu[:, :F]) * gu[:, F:]
    _close(z, z_ref, 2e-2)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
