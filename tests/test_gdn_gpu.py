"""GatedDeltaNet kernels against the fp32 eager forms."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _dev():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    return torch.device("cuda", 0)


@pytest.mark.parametrize("B,L,C,K,with_left", [(2, 37, 96, 4, True), (3, 5, 64, 4, False), (1, 2, 32, 2, True),
                                                (2, 64, 8192, 4, True)])
def test_conv_forward_backward(B, L, C, K, with_left):
    from ferrl_b200.models import gdn as G
    from ferrl_b200.ops import cuda as Cc
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(B + L + C)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    wide = rnd(B, L, C + 40).to(torch.bfloat16)
    x = wide[:, :, :C].detach().requires_grad_(True)          # strided view like the projection split
    w = (rnd(C, K) * 0.5).to(torch.bfloat16)
    left = rnd(B, C, K - 1).to(torch.bfloat16) if with_left else None
    y = Cc.gdn_conv(x, w, left, True)
    dy = rnd(B, L, C).to(torch.bfloat16)
    y.backward(dy)
    xr = x.detach().float().requires_grad_(True)
    yr, _ = G.causal_depthwise_conv1d(xr.transpose(1, 2), w.float(), None if left is None else left.float(), True)
    yr = yr.transpose(1, 2)
    yr.backward(dy.float())
    assert float((y.float() - yr).abs().max()) <= 0.02 * float(yr.abs().max()) + 1e-2
    assert float((x.grad.float() - xr.grad).abs().max()) <= 0.03 * float(xr.grad.abs().max()) + 1e-2


def test_conv_step_matches_prefill_and_shifts_state():
    from ferrl_b200.ops import cuda as Cc
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(4)
    B, C, K, L = 3, 128, 4, 9
    x = torch.randn(B, L, C, device=dev, generator=g).to(torch.bfloat16)
    w = (torch.randn(C, K, device=dev, generator=g) * 0.5).to(torch.bfloat16)
    full = Cc.gdn_conv(x, w, None, True)
    state = torch.zeros(B, C, K - 1, device=dev, dtype=torch.bfloat16)
    for t in range(L):
        y = Cc.gdn_conv_step(x[:, t], w, state, True)
        assert torch.equal(y, full[:, t])
    assert torch.equal(state, x[:, L - (K - 1):].transpose(1, 2))


@pytest.mark.parametrize("B,Hk,Hv,KD,VD", [(2, 2, 4, 128, 128), (3, 4, 4, 64, 64), (1, 1, 2, 32, 96)])
def test_decode_step_matches_recurrent(B, Hk, Hv, KD, VD):
    from ferrl_b200.models import gdn as G
    from ferrl_b200.ops import cuda as Cc
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(B + Hk + KD)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    S = rnd(B, Hv, KD, VD) * 0.1
    S_ref = S.clone()
    for step in range(3):
        q, k = rnd(B, Hk * KD).to(torch.bfloat16), rnd(B, Hk * KD).to(torch.bfloat16)
        v = rnd(B, Hv * VD).to(torch.bfloat16)
        gg = -torch.rand(B, Hv, device=dev, generator=g)
        beta = torch.rand(B, Hv, device=dev, generator=g)
        o = Cc.gdn_decode_step(q, k, v, gg, beta, S, True, 1e-6)
        rep = Hv // Hk
        qr = q.view(B, 1, Hk, KD).repeat_interleave(rep, dim=2).float()
        kr = k.view(B, 1, Hk, KD).repeat_interleave(rep, dim=2).float()
        o_ref, S_ref = G.gated_delta_rule_recurrent(qr, kr, v.view(B, 1, Hv, VD).float(), gg.view(B, 1, Hv),
                                                    beta.view(B, 1, Hv), S_ref, use_qk_l2norm=True)
        assert float((o.float() - o_ref[:, 0]).abs().max()) <= 0.02 * float(o_ref.abs().max()) + 1e-3
        assert float((S - S_ref).abs().max()) <= 1e-4 * float(S_ref.abs().max()) + 1e-5


def test_decode_step_with_gates_formed_in_the_kernel():
    """``gdn_decode_step_raw`` (g and beta from the projection's a / b columns, strided views) equals the step fed
    with gates computed by PyTorch."""
    import torch.nn.functional as F
    from ferrl_b200.ops import cuda as Cc
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(5)
    B, Hk, Hv, KD, VD = 5, 2, 4, 128, 128
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    S1 = rnd(B, Hv, KD, VD) * 0.1
    S2 = S1.clone()
    A_log = torch.log(torch.rand(Hv, device=dev, generator=g) * 15 + 1)
    dt_bias = rnd(Hv)
    for step in range(3):
        q, k = rnd(B, Hk * KD).to(torch.bfloat16), rnd(B, Hk * KD).to(torch.bfloat16)
        v = rnd(B, Hv * VD).to(torch.bfloat16)
        ab = (rnd(B, 2 * Hv + 3) * 3).to(torch.bfloat16)           # a and b as column slices of a wider row
        a, b = ab[:, 1:1 + Hv], ab[:, 1 + Hv:1 + 2 * Hv]
        gg = -A_log.exp() * F.softplus(a.float() + dt_bias)
        beta = torch.sigmoid(b.float())
        o1 = Cc.gdn_decode_step(q, k, v, gg, beta, S1, True, 1e-6)
        o2 = Cc.gdn_decode_step_raw(q, k, v, a, b, A_log, dt_bias, S2, True, 1e-6)
        assert float((o1.float() - o2.float()).abs().max()) <= 0.01 * float(o1.float().abs().max()) + 1e-3
        assert float((S1 - S2).abs().max()) <= 1e-4 * float(S1.abs().max()) + 1e-5


@pytest.mark.parametrize("B,T,Hk,Hv,with_state", [(1, 64, 1, 1, False), (2, 150, 2, 4, True), (1, 7, 1, 2, True),
                                                   (3, 257, 2, 2, False)])
def test_chunk_scan_matches_recurrent(B, T, Hk, Hv, with_state):
    """The chunked kernel (state in shared memory, 64-token chunks) against the token-by-token
    fp32 recurrence, including a ragged last chunk and a carried-in state."""
    from ferrl_b200.models import gdn as G
    from ferrl_b200.ops import cuda as Cc
    dev = _dev()
    g = torch.Generator(device=dev).manual_seed(B * 1000 + T)
    rnd = lambda *s: torch.randn(*s, device=dev, generator=g)
    q, k = rnd(B, T, Hk, 128).to(torch.bfloat16), rnd(B, T, Hk, 128).to(torch.bfloat16)
    v = rnd(B, T, Hv, 128).to(torch.bfloat16)
    gg = -torch.rand(B, T, Hv, device=dev, generator=g) * 0.5
    beta = torch.rand(B, T, Hv, device=dev, generator=g)
    S0 = rnd(B, Hv, 128, 128) * 0.05 if with_state else None
    out, S = Cc.gdn_chunk_fwd(q, k, v, gg, beta, S0, True, 1e-6)
    rep = Hv // Hk
    qr, kr = q.float().repeat_interleave(rep, dim=2), k.float().repeat_interleave(rep, dim=2)
    o_ref, S_ref = G.gated_delta_rule_recurrent(qr, kr, v.float(), gg, beta, S0, use_qk_l2norm=True)
    assert float((out.float() - o_ref).abs().max()) <= 0.02 * float(o_ref.abs().max()) + 1e-3
    assert float((S - S_ref).abs().max()) <= 2e-3 * float(S_ref.abs().max()) + 1e-4
    out2, S2 = Cc.gdn_chunk_fwd(q, k, v, gg, beta, S0, True, 1e-6)
    assert torch.equal(out, out2) and torch.equal(S, S2)
