"""Block-level goldens: GatedDeltaNet primitives, norm variants, partial-RoPE geometry, the MoE
router, expert dispatch (with experts no token reaches) and the whole sparse block against the
committed vectors generated from HF transformers (``tests/fixtures/gdn_golden.json``,
``moe_golden.json``)."""
import json
import os

import pytest
import torch
import torch.nn.functional as F

from ferrl_b200.models import gdn as G
from ferrl_b200.models import moe as M
from ferrl_b200.ops import eager as E

FIX = os.path.join(os.path.dirname(__file__), "fixtures")
GDN = json.load(open(os.path.join(FIX, "gdn_golden.json")))["cases"]
MOE = json.load(open(os.path.join(FIX, "moe_golden.json")))["cases"]
TOL = 2e-6


def T(c, key, *shape):
    return torch.tensor(c[key], dtype=torch.float32).reshape(*shape)


def err(a, b):
    return (a.float() - b.float()).abs().max().item()


@pytest.mark.parametrize("name", ["recurrent_no_state", "recurrent_with_state", "chunked_t130", "chunked_with_state"])
@pytest.mark.parametrize("form", ["recurrent", "chunked"])
def test_gated_delta_rule_both_forms_match_every_golden(name, form):
    """T=130 crosses two 64-token chunk boundaries with a ragged tail; the recurrent and the chunked
    form must both reproduce the reference output and final state, with and without a carried state."""
    c = GDN[name]
    b, t, h, k, v = (c[x] for x in "bthkv")
    st = T(c, "initial_state", b, h, k, v) if "initial_state" in c else None
    fn = G.gated_delta_rule_recurrent if form == "recurrent" else G.gated_delta_rule_chunked
    out, state = fn(T(c, "query", b, t, h, k), T(c, "key", b, t, h, k), T(c, "value", b, t, h, v), T(c, "g", b, t, h),
                    T(c, "beta", b, t, h), st, use_qk_l2norm=True)
    assert err(out, T(c, "out", b, t, h, v)) < TOL and err(state, T(c, "state", b, h, k, v)) < TOL
    wrong, _ = fn(T(c, "query", b, t, h, k), T(c, "key", b, t, h, k), T(c, "value", b, t, h, v), T(c, "g", b, t, h),
                  T(c, "beta", b, t, h), st, use_qk_l2norm=False)
    assert err(wrong, T(c, "out", b, t, h, v)) > 1e-2                    # negative control: the q/k normalisation matters


def test_conv_softplus_l2norm_and_norm_variants():
    for name in ("conv_no_ctx", "conv_with_ctx"):
        c = GDN[name]
        b, ch, l, K = c["b"], c["c"], c["l"], c["kernel"]
        left = T(c, "left", b, ch, K - 1) if "left" in c else None
        y, new_left = G.causal_depthwise_conv1d(T(c, "x", b, ch, l), T(c, "weight", ch, K), left)
        assert err(y, T(c, "out", b, ch, l)) < TOL
        assert torch.equal(new_left, T(c, "x", b, ch, l)[:, :, -(K - 1):])   # the context handed to the next call
    c = GDN["softplus"]
    assert err(G.stable_softplus(T(c, "x", -1)), T(c, "out", -1)) < TOL and err(E.stable_softplus(T(c, "x", -1)), T(c, "out", -1)) < TOL
    for name in ("l2norm", "l2norm_small"):
        c = GDN[name]
        x = T(c, "x", c["rows"], c["dim"])
        assert err(G.l2norm(x), T(c, "out", c["rows"], c["dim"])) < TOL and err(E.l2norm(x), T(c, "out", c["rows"], c["dim"])) < TOL
    c = GDN["rmsnorm_zero_centered"]
    sh = c["shape"]
    assert err(E.rmsnorm(T(c, "x", *sh), T(c, "weight", -1), 1e-6, zero_centered=True), T(c, "out", *sh)) < TOL
    assert err(E.rmsnorm(T(c, "x", *sh), T(c, "weight", -1), 1e-6, zero_centered=False), T(c, "out", *sh)) > 1e-2
    c = GDN["rmsnorm_gated"]
    r = c["rows"]
    assert err(E.rmsnorm_gated(T(c, "x", r, -1), T(c, "gate", r, -1), T(c, "weight", -1), 1e-6), T(c, "out", r, -1)) < TOL


def test_partial_rope_geometry_of_the_hybrid_family():
    """head_dim 256 with a 64-wide rotary span at theta 1e7: the other 192 channels pass through."""
    c = GDN["rope_text_qwen35_geometry"]
    l, D, rot = c["l"], c["head_dim"], c["rot_dim"]
    cos, sin = E.rope_tables(E.default_inv_freq(rot, c["rope_theta"]), 16)
    for name in ("q", "k"):
        x = T(c, name, 1, l, 1, D)
        y = E.apply_rope(x, cos, sin, torch.arange(l))
        assert err(y, T(c, name + "_out", 1, l, 1, D)) < TOL
        assert torch.equal(y[..., rot:], x[..., rot:])


@pytest.mark.parametrize("name", ["router_t5", "router_t1"])
def test_router_top_k(name):
    c = MOE[name]
    t, h, e, k = c["tokens"], c["hidden"], c["experts"], c["top_k"]
    x, w = T(c, "x", t, h), T(c, "weight", e, h)
    probs, scores, idx = M.topk_router(x, w, k)
    assert err(F.linear(x, w), T(c, "logits", t, e)) < TOL and err(scores, T(c, "scores", t, k)) < TOL
    assert torch.equal(idx, torch.tensor(c["indices"]).reshape(t, k))
    assert err(scores.sum(-1), torch.ones(t)) < 1e-6 and err(probs.sum(-1), torch.ones(t)) < 1e-6


@pytest.mark.parametrize("name", ["experts_t9", "experts_unhit_t2"])
def test_expert_dispatch_including_experts_no_token_reaches(name):
    c = MOE[name]
    t, h, e, k, i = c["tokens"], c["hidden"], c["experts"], c["top_k"], c["moe_inter"]
    idx = torch.tensor(c["indices"]).reshape(t, k)
    out = M.moe_experts(T(c, "x", t, h), idx, T(c, "scores", t, k), T(c, "gate_up_proj", e, 2 * i, h), T(c, "down_proj", e, h, i))
    assert err(out, T(c, "out", t, h)) < TOL
    if name == "experts_unhit_t2":
        assert len(set(idx.reshape(-1).tolist())) < e


@pytest.mark.parametrize("name", ["block_b1_t6", "block_b2_t4", "block_k1_b1_t3"])
def test_sparse_moe_block_with_gated_shared_expert(name):
    c = MOE[name]
    b, t, h, e, k, i, si = c["b"], c["t"], c["hidden"], c["experts"], c["top_k"], c["moe_inter"], c["shared_inter"]
    sg, su, sd = T(c, "shared_gate_proj", si, h), T(c, "shared_up_proj", si, h), T(c, "shared_down_proj", h, si)

    def shared(x):
        return F.linear(F.silu(F.linear(x, sg)) * F.linear(x, su), sd)
    out = M.sparse_moe_block(T(c, "x", b, t, h), T(c, "router_weight", e, h), T(c, "gate_up_proj", e, 2 * i, h),
                             T(c, "down_proj", e, h, i), k, shared=shared, shared_gate_w=T(c, "shared_expert_gate", 1, h))
    assert err(out, T(c, "out", b, t, h)) < 5e-6


def test_lora_scale_must_survive_the_base_compute_dtype():
    """crates/ferrl/src/lora.rs:1597-1632 as golden cases: alpha / rank is checked in the dtype the frozen base
    computes in, with closed ranges for the 16-bit types."""
    import sys

    import pytest
    import torch

    from ferrl_b200.models.lora import FusedLoraLinear, LoraSpec, validated_lora_scale
    for dtype in (torch.float32, torch.bfloat16):
        assert validated_lora_scale(2, 8.0, dtype) == 4.0
        for alpha in (sys.float_info.min, sys.float_info.max):
            with pytest.raises(ValueError, match="lora scale"):
                validated_lora_scale(2, alpha, dtype)
    for scale in (5.960464477539063e-8, 1.0, 65504.0):
        assert validated_lora_scale(1, scale, torch.float16) == scale
    for scale in (5.960464477539063e-8 / 2.0, 65536.0):
        with pytest.raises(ValueError, match="compute dtype F16"):
            validated_lora_scale(1, scale, torch.float16)
    with pytest.raises(ValueError, match="rank must be > 0"):
        validated_lora_scale(0, 8.0)
    for alpha in (0.0, -1.0, float("nan"), float("inf")):
        with pytest.raises(ValueError, match="alpha must be finite and > 0"):
            validated_lora_scale(2, alpha)
    # a scale that float32 can hold but bfloat16 cannot: the constructor checks in the base's dtype
    tiny = LoraSpec(1, 1e-42)
    FusedLoraLinear(3, [4], ("p",), (True,), tiny, dtype=torch.float32)
    with pytest.raises(ValueError, match="compute dtype BF16"):
        FusedLoraLinear(3, [4], ("p",), (True,), tiny, dtype=torch.bfloat16)


def test_chunked_delta_rule_survives_cumulative_decay_underflow():
    """crates/ferrl/src/gdn.rs:1062-1081: with log-decays near -2.3 per step the cumulative decay of a 64-token chunk
    underflows float32 (exp(-150)); the chunked form must still equal the recurrence and stay finite, within a chunk
    and with the state carried across chunks."""
    import torch

    from ferrl_b200.models import gdn as G
    gen = torch.Generator().manual_seed(71)
    for t in (64, 200):
        q, k = torch.randn(1, t, 1, 3, generator=gen), torch.randn(1, t, 1, 3, generator=gen)
        v = torch.randn(1, t, 1, 3, generator=gen)
        beta = torch.sigmoid(torch.randn(1, t, 1, generator=gen))
        g = -(2.2 + 0.3 * torch.rand(1, t, 1, generator=gen))
        for l2 in (False, True):
            o_r, s_r = G.gated_delta_rule_recurrent(q, k, v, g, beta, None, use_qk_l2norm=l2)
            o_c, s_c = G.gated_delta_rule_chunked(q, k, v, g, beta, None, use_qk_l2norm=l2)
            assert torch.isfinite(o_c).all() and torch.isfinite(s_c).all()
            assert float((o_r - o_c).abs().max()) <= 2e-5 and float((s_r - s_c).abs().max()) <= 2e-5
