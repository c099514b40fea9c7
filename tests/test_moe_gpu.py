"""Device-resident mixture-of-experts path against the eager plan in fp32."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("T,E,k", [(77, 8, 2), (1000, 64, 8), (5, 128, 4), (300, 200, 6)])
def test_route_matches_softmax_topk(T, E, k):
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(T + E)
    logits = torch.randn(T, E, device=dev, generator=g) * 3
    logits.requires_grad_(True)
    scores, idx, counts, probs = C.moe_route(logits, k, True)
    ref = torch.softmax(logits.detach().double(), -1)
    assert float((probs.double() - ref).abs().max()) < 1e-6
    top = torch.topk(ref, k, dim=-1)
    want = top.values / top.values.sum(-1, keepdim=True)
    # equal probabilities may be ordered differently; the values are what must agree
    assert float((scores.double() - want).abs().max()) < 1e-5
    assert float((ref.gather(1, idx.long()) - top.values).abs().max()) < 1e-6
    assert torch.equal(counts.long(), torch.bincount(idx.flatten().long(), minlength=E))
    # backward against autograd through the same selection
    w = torch.randn(T, k, device=dev, generator=g)
    (scores * w).sum().backward()
    l2 = logits.detach().clone().requires_grad_(True)
    p2 = torch.softmax(l2, -1).gather(1, idx.long())
    ((p2 / p2.sum(-1, keepdim=True)) * w).sum().backward()
    assert float((logits.grad - l2.grad).abs().max()) < 1e-5


@pytest.mark.parametrize("T,E,k,H,I", [(200, 8, 2, 128, 256), (1500, 32, 4, 256, 128), (3, 16, 2, 128, 128)])
def test_experts_forward_backward(T, E, k, H, I):
    from ferrl_b200.models import moe as M
    from ferrl_b200.ops import cuda as C
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(T + E + H)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    x = rnd(T, H).to(torch.bfloat16).requires_grad_(True)
    gate_up = (rnd(E, 2 * I, H) / H ** 0.5).to(torch.bfloat16)
    down = (rnd(E, H, I) / I ** 0.5).to(torch.bfloat16)
    logits = rnd(T, E)
    scores, idx, counts, _ = C.moe_route(logits, k, True)
    scores = scores.detach().requires_grad_(True)
    y = C.moe_experts(x, scores, idx, counts, gate_up, down, "silu")
    assert C.kernel_status() == 0
    dy = rnd(T, H).to(torch.bfloat16)
    y.backward(dy)

    xr = x.detach().float().requires_grad_(True)
    sr = scores.detach().clone().requires_grad_(True)
    yr = M.moe_experts(xr, idx.long(), sr, gate_up.float(), down.float(), "silu")
    yr.backward(dy.float())
    tol = lambda ref: 0.03 * float(ref.abs().max()) + 1e-3
    assert float((y.float() - yr).abs().max()) <= tol(yr)
    assert float((x.grad.float() - xr.grad).abs().max()) <= tol(xr.grad)
    assert float((scores.grad - sr.grad).abs().max()) <= tol(sr.grad)
    # transposed resident copies give the same gradients
    x2 = x.detach().clone().requires_grad_(True)
    y2 = C.moe_experts(x2, scores.detach(), idx, counts, gate_up, down, "silu",
                       gate_up.transpose(1, 2).contiguous(), down.transpose(1, 2).contiguous())
    y2.backward(dy)
    assert torch.equal(y2, y) and torch.equal(x2.grad, x.grad)


def test_block_is_deterministic_and_matches_eager():
    from ferrl_b200.models import moe as M
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(9)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    T, E, k, H, I = 513, 16, 4, 128, 128
    x = rnd(2, T, H).to(torch.bfloat16)
    router = rnd(E, H).to(torch.bfloat16)
    gate_up = (rnd(E, 2 * I, H) / H ** 0.5).to(torch.bfloat16)
    down = (rnd(E, H, I) / I ** 0.5).to(torch.bfloat16)
    a = M.sparse_moe_block(x, router, gate_up, down, k)
    b = M.sparse_moe_block(x, router, gate_up, down, k)
    assert torch.equal(a, b)
    ref = M.sparse_moe_block(x.cpu().float(), router.cpu().float(), gate_up.cpu().float(), down.cpu().float(), k)
    # routing on bf16 logits can pick a different expert on near-ties; almost every row must agree
    err = (a.cpu().float() - ref).abs().amax(-1).flatten()
    assert float((err <= 0.05 * float(ref.abs().max())).float().mean()) > 0.97


def test_expert_parallel_world1_equals_local_plan():
    """With one rank the dispatch/combine kernels must reproduce the local plan exactly."""
    from ferrl_b200.comm import SoloComm
    from ferrl_b200.ops import cuda as C
    from ferrl_b200.parallel.ep import EpRuntime
    from ferrl_b200.parallel.symm import SymmHeap
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(21)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    T, E, k, H, I = 700, 16, 4, 256, 128
    gate_up = (rnd(E, 2 * I, H) / H ** 0.5).to(torch.bfloat16)
    down = (rnd(E, H, I) / I ** 0.5).to(torch.bfloat16)
    scores, idx, counts, _ = C.moe_route(rnd(T, E), k, True)
    dy = rnd(T, H).to(torch.bfloat16)
    rt = EpRuntime(SymmHeap(SoloComm(), dev, wait_limit_s=1.0), E, H, T, k)
    outs = []
    for fn in (lambda x, s: C.moe_experts(x, s, idx, counts, gate_up, down, "silu"),
               lambda x, s: rt.experts(x, s, idx, counts, gate_up, down, "silu")):
        x = rnd(T, H).to(torch.bfloat16) if not outs else outs[0][3]
        x = x.detach().clone().requires_grad_(True)
        s = scores.detach().clone().requires_grad_(True)
        y = fn(x, s)
        y.backward(dy)
        outs.append((y.detach(), x.grad, s.grad, x.detach()))
    assert C.kernel_status() == 0
    assert torch.equal(outs[0][0], outs[1][0])
    assert torch.equal(outs[0][1], outs[1][1])
    assert torch.equal(outs[0][2], outs[1][2])
