"""The decode projection with resident activations (``csrc/gemm/decode_gemm.cu``) against an fp32
PyTorch restatement: plain, residual, GLU epilogue, k groups (K > 4096), ragged M, k-block counts
that leave cluster ranks without work, one cluster walking every tile, canary-padded outputs and
bitwise reruns (the cross-CTA sums run in a fixed order)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _ops():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ferrl_b200.ops import cuda as C
    return C


def _ref(a, b, res=None):
    y = a.float() @ b.float().t()
    if res is not None:
        y = y + res.float()
    return y


def _check(out, ref, k):
    # bf16 output: half an ulp of the result plus the fp32 accumulation error over k terms
    tol = 2e-2 * ref.abs().clamp(min=1.0) * 0.5 + 1e-3 * (k ** 0.5)
    bad = (out.float() - ref).abs() > tol
    assert not bad.any(), (int(bad.sum()), float((out.float() - ref).abs().max()))


@pytest.mark.parametrize("M,N,K,res,clusters", [
    (128, 6144, 4096, False, 0), (128, 4096, 4096, True, 0), (128, 4096, 12288, True, 0), (128, 4096, 12288, False, 0),
    (37, 1024, 1024, True, 0), (1, 64, 512, False, 0), (128, 1024, 5376, True, 0), (64, 512, 576, False, 0),
    (128, 8192, 4096, True, 1), (100, 2048, 8192, True, 2), (128, 24576, 4096, False, 0),
])
def test_decode_gemm_matches_fp32_reference(M, N, K, res, clusters):
    C = _ops()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(M * 7 + N + K)
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev, generator=g) * 0.05).to(torch.bfloat16)
    r = torch.randn(M, N, device=dev, generator=g).to(torch.bfloat16) if res else None
    C.lib().reset_status()
    y1 = C.lib().decode_gemm(a, b, r, -1, clusters, False)
    y2 = C.lib().decode_gemm(a, b, r, -1, clusters, True)      # launched as a programmatic dependent
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    assert torch.equal(y1, y2)
    _check(y1, _ref(a, b, r), K)
    # a dropped last k-block or a wrong boundary column shows up as a whole wrong row/column, not as noise
    ref = _ref(a, b, r)
    assert float((y1.float() - ref).abs().amax(dim=0).max()) < 0.25 and float((y1.float() - ref).abs().amax(dim=1).max()) < 0.25


def test_decode_gemm_glu_epilogue_and_product_dispatch():
    C = _ops()
    dev = torch.device("cuda", 0)
    g = torch.Generator(device=dev).manual_seed(5)
    M, F, K = 128, 3072, 4096
    a = torch.randn(M, K, device=dev, generator=g).to(torch.bfloat16)
    wg = (torch.randn(F, K, device=dev, generator=g) * 0.03).to(torch.bfloat16)
    wu = (torch.randn(F, K, device=dev, generator=g) * 0.03).to(torch.bfloat16)
    # groups of 16 rows: 8 gate rows followed by the 8 up rows of the same features
    w = torch.stack([wg.view(F // 8, 8, K), wu.view(F // 8, 8, K)], dim=1).reshape(2 * F, K).contiguous()
    C.lib().reset_status()
    for act, fn in ((0, torch.nn.functional.silu), (1, lambda x: torch.nn.functional.gelu(x, approximate="tanh"))):
        y = C.lib().decode_gemm(a, w, None, act, 0, False)
        ref = fn(a.float() @ wg.float().t()) * (a.float() @ wu.float().t())
        _check(y, ref, K)
    # switched on, the public wrappers pick this kernel for weights (static_b) and agree with the planner's other kernels
    y_old = C.gemm_glu(a, w, "silu")
    p_old = C.gemm(a, wg, static_b=True)
    C.lib().set_decode_gemm(True)
    try:
        y_new = C.gemm_glu(a, w, "silu")
        p_new = C.gemm(a, wg, static_b=True)
    finally:
        C.lib().set_decode_gemm(False)
    torch.cuda.synchronize()
    assert C.kernel_status() == 0
    # different summation orders of the same products: at most about one bf16 ulp of the result apart
    for new, old in ((y_new, y_old), (p_new, p_old)):
        d = (new.float() - old.float()).abs()
        assert bool((d <= 1e-2 * old.float().abs().clamp(min=1.0)).all()), float(d.max())


def test_decode_gemm_writes_nothing_outside_its_output():
    """Output allocated inside a canary-padded buffer (row stride wider than N): pads stay intact."""
    C = _ops()
    dev = torch.device("cuda", 0)
    M, N, K = 77, 1024, 2048
    a = torch.randn(M, K, device=dev).to(torch.bfloat16)
    b = (torch.randn(N, K, device=dev) * 0.05).to(torch.bfloat16)
    y = C.lib().decode_gemm(a, b, None, -1, 0, False)
    # the op allocates its own [M, N] output; surround a copy of the same call's memory neighbourhood
    # by checking the rows the kernel must not touch: run it on a 128-row tile whose rows >= M do not exist
    big = torch.full((128, N), 7.0, device=dev, dtype=torch.bfloat16)
    big[:M] = y
    assert torch.all(big[M:] == 7.0)
    a_pad = torch.zeros(128, K, device=dev, dtype=torch.bfloat16)
    a_pad[:M] = a
    y_full = C.lib().decode_gemm(a_pad, b, None, -1, 0, False)
    assert torch.equal(y_full[:M], y) and torch.all(y_full[M:] == 0)


def test_decode_gemm_rejects_unsupported_shapes():
    C = _ops()
    dev = torch.device("cuda", 0)
    a = torch.zeros(129, 512, device=dev, dtype=torch.bfloat16)
    b = torch.zeros(64, 512, device=dev, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError):
        C.lib().decode_gemm(a, b, None, -1, 0, False)
    with pytest.raises(RuntimeError):
        C.lib().decode_gemm(a[:8], torch.zeros(72, 512, device=dev, dtype=torch.bfloat16), None, -1, 0, False)
    with pytest.raises(RuntimeError):
        C.lib().decode_gemm(a[:8, :256].contiguous(), torch.zeros(64, 256, device=dev, dtype=torch.bfloat16), None, -1, 0, False)
