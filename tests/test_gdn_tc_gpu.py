"""Tensor-core chunked gated delta rule (forward and hand-written backward) and the gated RMSNorm
backward, against the token-by-token recurrence in float64 and autograd through it.

Reference behaviour: crates/ferrl/src/gdn.rs:451-556 (chunked form) must equal the recurrent form."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _recurrent(q, k, v, g, beta, S):
    """float64 recurrence; q,k already L2-normalised and q scaled."""
    outs = []
    for t in range(q.shape[1]):
        S = S * g[:, t].exp()[..., None, None]
        kv = (S * k[:, t].unsqueeze(-1)).sum(-2)
        delta = (v[:, t] - kv) * beta[:, t].unsqueeze(-1)
        S = S + k[:, t].unsqueeze(-1) * delta.unsqueeze(-2)
        outs.append((S * q[:, t].unsqueeze(-1)).sum(-2))
    return torch.stack(outs, 1), S


def _rel(a, b):
    return ((a.double() - b.double()).norm() / b.double().norm().clamp_min(1e-12)).item()


# the last case has enough (batch, head) pairs for the 64-column scan slices; the others take the 32-column ones
@pytest.mark.parametrize("B,T,Hk,Hv,with_state", [(2, 128, 2, 2, False), (1, 130, 1, 2, True), (2, 64, 2, 4, True),
                                                   (2, 192, 20, 40, True)])
def test_gdn_tc_matches_recurrence_with_grads(B, T, Hk, Hv, with_state):
    from ferrl_b200.ops import cuda as C, eager
    dev = torch.device("cuda")
    torch.manual_seed(T + Hv)
    D = 128
    q = torch.randn(B, T, Hk, D, device=dev)
    k = torch.randn(B, T, Hk, D, device=dev)
    v = torch.randn(B, T, Hv, D, device=dev)
    g = -torch.rand(B, T, Hv, device=dev) * 0.3
    beta = torch.rand(B, T, Hv, device=dev) * 0.9 + 0.05
    S0 = torch.randn(B, Hv, D, D, device=dev) * 0.05 if with_state else None
    leaves = [t.clone().requires_grad_() for t in (q, k, v, g, beta)] + ([S0.clone().requires_grad_()] if with_state else [])
    out, S1 = C.gdn_chunk_tc(*leaves[:5], leaves[5] if with_state else None)
    dO, dS1 = torch.randn_like(out), torch.randn_like(S1) * 0.1
    ((out * dO).sum() + (S1 * dS1).sum()).backward()
    got = [t.grad for t in leaves]

    ref_leaves = [t.double().clone().requires_grad_() for t in (q, k, v, g, beta)] + \
        ([S0.double().clone().requires_grad_()] if with_state else [])
    rq, rk, rv, rg, rb = ref_leaves[:5]
    rep = Hv // Hk
    qn = (eager.l2norm(rq, 1e-6) * D ** -0.5).repeat_interleave(rep, dim=2)
    kn = eager.l2norm(rk, 1e-6).repeat_interleave(rep, dim=2)
    S = ref_leaves[5] if with_state else torch.zeros(B, Hv, D, D, device=dev, dtype=torch.float64)
    ro, rS = _recurrent(qn, kn, rv, rg, rb, S)
    ((ro * dO.double()).sum() + (rS * dS1.double()).sum()).backward()
    assert _rel(out, ro) < 4e-3, _rel(out, ro)
    assert _rel(S1, rS) < 4e-3, _rel(S1, rS)
    for name, a, r in zip(["q", "k", "v", "g", "beta", "S0"], got, [t.grad for t in ref_leaves]):
        assert a is not None and torch.isfinite(a).all(), name
        assert _rel(a, r) < 1e-2, (name, _rel(a, r))


def test_gdn_tc_forward_without_grad_matches_the_scan_kernel():
    from ferrl_b200.ops import cuda as C
    dev = torch.device("cuda")
    torch.manual_seed(0)
    q, k = torch.randn(1, 64, 2, 128, device=dev), torch.randn(1, 64, 2, 128, device=dev)
    v = torch.randn(1, 64, 2, 128, device=dev, dtype=torch.bfloat16)
    g, beta = -torch.rand(1, 64, 2, device=dev) * 0.2, torch.rand(1, 64, 2, device=dev)
    with torch.no_grad():
        out, S1 = C.gdn_chunk_tc(q, k, v, g, beta)
        ref = C.gdn_chunk_fwd(q.bfloat16(), k.bfloat16(), v, g, beta, None, True, 1e-6)
    assert out.dtype == torch.bfloat16 and S1.dtype == torch.float32
    assert _rel(out.float(), ref[0].float()) < 2e-2
    assert _rel(S1, ref[1]) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_rmsnorm_gated_backward(dtype):
    from ferrl_b200.ops import cuda as C, eager
    dev = torch.device("cuda")
    torch.manual_seed(1)
    x = torch.randn(777, 128, device=dev).to(dtype)
    gate = torch.randn(777, 128, device=dev).to(dtype)
    w = (torch.rand(128, device=dev) + 0.5).to(dtype)
    dy = torch.randn(777, 128, device=dev).to(dtype)
    xs, gs = x.clone().requires_grad_(), gate.clone().requires_grad_()
    y = C.rmsnorm_gated(xs, gs, w, 1e-6)
    y.backward(dy)
    xr, gr = x.double().requires_grad_(), gate.double().requires_grad_()
    yr = eager.rmsnorm_gated(xr, gr, w.double(), 1e-6)
    yr.backward(dy.double())
    tol = 2e-5 if dtype == torch.float32 else 1e-2
    assert _rel(y, yr) < tol
    assert _rel(xs.grad, xr.grad) < tol and _rel(gs.grad, gr.grad) < tol
