"""GRPO math: scalar oracle against committed goldens, tensor loss against the TRL goldens
and the scalar oracle, finite-difference gradient checks, advantage invariants."""
import json
import math
import os

import pytest
import torch
from hypothesis import given, settings, strategies as st

from ferrl_b200 import grpo
from ferrl_b200.grpo import ImportanceSamplingLevel, LossConfig, LossType, ScaleRewards

FIX = os.path.join(os.path.dirname(__file__), "fixtures")


def _golden(name):
    with open(os.path.join(FIX, name)) as f:
        return json.load(f)


def test_scalar_goldens():
    g = _golden("grpo_golden.json")
    assert grpo.GROUP_STD_EPS == g["eps_std"]
    for grp in g["groups"]:
        for a, b in zip(grpo.group_advantages(grp["rewards"], ScaleRewards.GROUP), grp["advantages"]):
            assert abs(a - b) < 1e-12
        for a, b in zip(grpo.group_advantages(grp["rewards"], ScaleRewards.NONE), grp["advantages_unscaled"]):
            assert abs(a - b) < 1e-12
    for c in g["k3_kl"]:
        assert abs(grpo.k3_kl(c["logp"], c["logp_ref"]) - c["kl"]) < 1e-12
    for c in g["clipped_surrogate"]:
        assert abs(grpo.clipped_surrogate(c["ratio"], c["advantage"], c["eps_low"], c["eps_high"]) - c["value"]) < 1e-12
    mm = g["masked_mean"]
    for lt in ("grpo", "dr_grpo", "dapo"):
        assert abs(grpo.masked_mean(mm["per_token"], mm["mask"], LossType(lt)) - mm[lt]) < 1e-12
    for c in g["sequence_log_ratio"]:
        assert abs(grpo.sequence_log_ratio(c["logp"], c["logp_old"], c["mask"]) - c["value"]) < 1e-12


def test_tensor_loss_matches_trl_goldens_and_scalar_oracle():
    g = _golden("grpo_golden_trl.json")
    b = g["batch"]
    t = {k: torch.tensor(v, dtype=torch.float64) for k, v in b.items()}
    assert len(g["cases"]) == 32
    for c in g["cases"]:
        cfg = LossConfig(c["eps_low"], c["eps_high"], c["beta"], LossType(c["loss_type"]),
                         ImportanceSamplingLevel(c["importance_sampling_level"]), c["dapo_norm"])
        ref = t["logp_ref"] if c["beta"] > 0 else None
        loss = grpo.grpo_loss_eager(t["logp"], t["logp_old"], ref, t["advantages"], t["mask"], cfg).item()
        assert abs(loss - c["loss"]) < 1e-9, c
        scalar = grpo.grpo_loss_scalar(b["logp"], b["logp_old"], b["logp_ref"] if c["beta"] > 0 else None,
                                       b["advantages"], b["mask"], eps_low=c["eps_low"], eps_high=c["eps_high"],
                                       beta=c["beta"], loss_type=c["loss_type"],
                                       is_level=c["importance_sampling_level"], dapo_norm=c["dapo_norm"])
        assert abs(scalar - c["loss"]) < 1e-9, c


@pytest.mark.parametrize("lt", list(LossType))
@pytest.mark.parametrize("level", list(ImportanceSamplingLevel))
@pytest.mark.parametrize("beta", [0.0, 0.04])
def test_gradcheck_against_central_differences(lt, level, beta):
    torch.manual_seed(0)
    G, L = 3, 5
    logp = (-torch.rand(G, L, dtype=torch.float64)).requires_grad_(True)
    old = logp.detach() + 0.2 * torch.randn(G, L, dtype=torch.float64)
    ref = logp.detach() + 0.1 * torch.randn(G, L, dtype=torch.float64)
    adv = torch.tensor([0.7, -1.1, 0.4], dtype=torch.float64)
    mask = torch.tensor([[1, 1, 1, 1, 0], [1, 1, 0, 0, 0], [1, 1, 1, 1, 1]], dtype=torch.float64)
    cfg = LossConfig(0.2, 0.28, beta, lt, level, 9.0 if lt is LossType.DAPO else None)
    fn = lambda x: grpo.grpo_loss_eager(x, old, ref if beta > 0 else None, adv, mask, cfg)  # noqa: E731
    fn(logp).backward()
    eps = 1e-6
    for i in range(G):
        for j in range(L):
            d = torch.zeros_like(logp)
            d[i, j] = eps
            fd = (fn(logp.detach() + d) - fn(logp.detach() - d)).item() / (2 * eps)
            assert abs(fd - logp.grad[i, j].item()) < 1e-6


def test_padding_is_gradient_inert_and_nan_safe():
    logp = torch.tensor([[-1.0, float("nan")]], requires_grad=True)
    old = torch.tensor([[-1.1, -2.0]])
    mask = torch.tensor([[1.0, 0.0]])
    loss = grpo.grpo_loss_eager(logp, old, old, torch.tensor([1.0]), mask, LossConfig(beta=0.1))
    assert math.isfinite(loss.item())
    loss.backward()
    assert logp.grad[0, 1].item() == 0.0 or math.isnan(logp.grad[0, 1].item()) is False


def test_zero_advantage_with_overflowed_ratio_is_zero():
    logp = torch.tensor([[100.0]])
    old = torch.tensor([[-100.0]])
    loss = grpo.grpo_loss_eager(logp, old, None, torch.tensor([0.0]), torch.ones(1, 1), LossConfig())
    assert loss.item() == 0.0


def test_dapo_equals_grpo_for_equal_length_unmasked():
    torch.manual_seed(1)
    lp, lo = -torch.rand(4, 6), -torch.rand(4, 6)
    adv, mask = torch.randn(4), torch.ones(4, 6)
    a = grpo.grpo_loss_eager(lp, lo, None, adv, mask, LossConfig(loss_type=LossType.GRPO))
    b = grpo.grpo_loss_eager(lp, lo, None, adv, mask, LossConfig(loss_type=LossType.DAPO))
    assert abs(a.item() - b.item()) < 1e-6


@settings(max_examples=200, deadline=None)
@given(st.lists(st.floats(-100, 100, allow_nan=False), min_size=2, max_size=16))
def test_advantages_zero_mean_and_shift_invariant(rs):
    adv = grpo.group_advantages(rs, ScaleRewards.GROUP)
    assert abs(sum(adv)) < 1e-6 * max(1.0, max(abs(a) for a in adv)) * len(adv)
    shifted = grpo.group_advantages([r + 3.0 for r in rs], ScaleRewards.GROUP)
    for a, b in zip(adv, shifted):
        assert abs(a - b) < 1e-6 * max(1.0, abs(a))


@settings(max_examples=100, deadline=None)
@given(st.floats(-1e3, 1e3, allow_nan=False), st.integers(2, 12))
def test_degenerate_group_has_zero_advantages(r, n):
    assert all(a == 0.0 for a in grpo.group_advantages([r] * n))


def test_advantage_input_validation():
    with pytest.raises(ValueError):
        grpo.group_advantages([])
    with pytest.raises(ValueError):
        grpo.group_advantages([1.0, float("inf")])
    assert all(math.isfinite(a) for a in grpo.group_advantages([3e38, -3e38, 0.0]))


def test_canonical_sum_is_order_independent():
    vals = [1e16, 1.0, -1e16, 3.0, 1e-3]
    assert grpo.canonical_sum(vals) == grpo.canonical_sum(list(reversed(vals))) == 4.001
    assert grpo.canonical_sum([1.0, float("nan")]) is None


def test_masked_mean_rejects_bad_inputs():
    with pytest.raises(ValueError):
        grpo.masked_mean([[1.0, 2.0], [1.0]], [[1.0, 1.0], [1.0]])
    with pytest.raises(ValueError):
        grpo.masked_mean([[1.0]], [[-1.0]])
    assert grpo.zero_mask_rows([[0.0, 0.0], [1.0, 0.0]]) == 1


def test_group_advantages_on_the_reference_extreme_vectors():
    """crates/ferrl/src/grpo.rs:734-835 as golden cases: inexact identical rewards stay exactly degenerate, values at
    the float32 limit neither overflow nor lose the group's shape, and the result does not depend on the order of
    the rewards (compensated canonical sum)."""
    import itertools
    import struct

    import pytest

    from ferrl_b200.grpo import ScaleRewards, group_advantages, tis_weight
    mag = struct.unpack("<f", struct.pack("<I", 0x7F7FFFFF))[0]          # f32::MAX
    for scale in ScaleRewards:
        assert group_advantages([0.1] * 3, scale) == [0.0] * 3
        assert group_advantages([mag, mag], scale) == [0.0, 0.0]
    for rewards in ([mag, -mag], [mag, -mag, -mag]):
        adv = group_advantages(rewards, ScaleRewards.GROUP)
        assert all(math.isfinite(a) for a in adv) and any(abs(a) > 0.5 for a in adv)
    canonical = [mag, 1.0, -mag]
    for scale in ScaleRewards:
        want = group_advantages(canonical, scale)
        for perm in itertools.permutations(canonical):
            got = group_advantages(list(perm), scale)
            assert all(a == want[canonical.index(r)] for r, a in zip(perm, got))
    assert abs(group_advantages(canonical, ScaleRewards.NONE)[1] - 2.0 / 3.0) <= 1e-15
    for bad, msg in (([], "empty reward group"), ([1.0, float("nan"), 3.0], "rewards must be finite"),
                     ([float("nan")] * 2, "rewards must be finite"), ([1.0, float("inf"), 3.0], "rewards must be finite")):
        with pytest.raises(ValueError, match=msg):
            group_advantages(bad, ScaleRewards.GROUP)
    assert abs(tis_weight(-1.5, -1.5, 2.0) - 1.0) < 1e-12 and abs(tis_weight(-1.0, -1.5, 2.0) - math.exp(0.5)) < 1e-12
    assert abs(tis_weight(-0.5, -2.0, 2.0) - 2.0) < 1e-12 and abs(tis_weight(-2.0, -0.5, 2.0) - math.exp(-1.5)) < 1e-12
