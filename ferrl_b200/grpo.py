"""GRPO objective math: group-relative advantages, clipped surrogate, k3 KL,
truncated importance sampling and the three loss reductions.

Two layers live here:

* a scalar float64 host oracle (``group_advantages``, ``k3_kl``,
  ``clipped_surrogate``, ``tis_weight``, ``masked_mean`` ...) that the trainer
  uses for advantages and that tests use as ground truth;
* a differentiable tensor loss (``grpo_loss``) over ``[G, L]`` log-prob
  matrices.  On CUDA tensors it runs the fused sm_100a kernel from
  ``ferrl_b200.ops`` (one launch forward, one backward); on CPU it runs the
  eager restatement below, which is also the kernel's numerical oracle.

Behavioural parity: reference ``crates/ferrl/src/grpo.rs:56-566`` (scalar
math) and ``crates/ferrl/src/trainer.rs:9788-9985`` (tensor loss).
"""
from __future__ import annotations

import enum
import math
from dataclasses import dataclass
from typing import Optional, Sequence

import torch

GROUP_STD_EPS = 1e-4
MAX_REWARD_MAGNITUDE = float(torch.finfo(torch.float32).max)
RATIO_LOG_CAP = 60.0


class LossType(str, enum.Enum):
    """Reduction over the per-token objective (reference grpo.rs:61-87)."""

    GRPO = "grpo"
    DR_GRPO = "dr_grpo"
    DAPO = "dapo"


class ScaleRewards(str, enum.Enum):
    GROUP = "group"
    NONE = "none"


class ImportanceSamplingLevel(str, enum.Enum):
    TOKEN = "token"
    SEQUENCE = "sequence"  # GSPO


# --------------------------------------------------------------------------
# scalar float64 oracle
# --------------------------------------------------------------------------

def canonical_sum(values: Sequence[float]) -> Optional[float]:
    """Order-independent correctly-rounded sum (``math.fsum``); ``None`` when an
    input is non-finite or the exact sum overflows.  Every rank obtains the same
    bits regardless of the order in which it saw the addends."""
    vals = list(values)
    if not all(math.isfinite(v) for v in vals):
        return None
    try:
        s = math.fsum(vals)
    except OverflowError:
        return None
    return s if math.isfinite(s) else None


@dataclass(frozen=True)
class FiniteMoments:
    """Mean and centred second moment of a reward group, computed on values
    pre-divided by ``scale`` (the largest magnitude) so neither the sum nor the
    squares overflow for rewards near the float32 limit."""

    count: int
    scale: float
    mean_scaled: float
    m2_scaled: float

    @property
    def mean(self) -> float:
        return self.mean_scaled * self.scale

    def sample_std(self) -> float:
        if self.count < 2:
            return 0.0
        return math.sqrt(self.m2_scaled / (self.count - 1)) * self.scale

    def population_std(self) -> float:
        if self.count == 0:
            return 0.0
        return math.sqrt(self.m2_scaled / self.count) * self.scale

    def centered(self, value: float) -> float:
        return value - self.mean

    def group_scaled(self, value: float) -> float:
        std = self.sample_std()
        out = (value - self.mean) / (std + GROUP_STD_EPS)
        if math.isfinite(out) and math.isfinite(std):
            return out
        sstd = 0.0 if self.count < 2 else math.sqrt(self.m2_scaled / (self.count - 1))
        return (value / self.scale - self.mean_scaled) / (sstd + GROUP_STD_EPS / self.scale)


def finite_moments(values: Sequence[float]) -> FiniteMoments:
    vals = [float(v) for v in values]
    n = len(vals)
    if n == 0:
        return FiniteMoments(0, 0.0, 0.0, 0.0)
    scale = max(abs(v) for v in vals)
    if scale == 0.0:
        return FiniteMoments(n, 0.0, 0.0, 0.0)
    if min(vals) == max(vals):  # degenerate group: exact mean, exactly zero spread
        return FiniteMoments(n, 1.0, vals[0], 0.0)
    # Rewards that are O(1) keep scale == 1 so ordinary arithmetic is bit-equal to
    # the plain numpy ddof=1 computation.
    scale = scale if scale > 1e150 else 1.0
    scaled = [v / scale for v in vals]
    mean = math.fsum(scaled) / n
    m2 = math.fsum((v - mean) * (v - mean) for v in scaled)
    return FiniteMoments(n, scale, mean, m2)


def group_advantages(rewards: Sequence[float], scale: ScaleRewards = ScaleRewards.GROUP) -> list[float]:
    """``A_i = (r_i - mean) / (std_ddof1 + 1e-4)`` (or just centred)."""
    if len(rewards) == 0:
        raise ValueError("group_advantages: empty reward group")
    if not all(math.isfinite(r) for r in rewards):
        raise ValueError("group_advantages: rewards must be finite")
    if not all(abs(r) <= MAX_REWARD_MAGNITUDE for r in rewards):
        raise ValueError("group_advantages: rewards must be within the float32 range")
    m = finite_moments(rewards)
    scale = ScaleRewards(scale)
    if scale is ScaleRewards.NONE:
        return [m.centered(float(r)) for r in rewards]
    return [m.group_scaled(float(r)) for r in rewards]


def advantages_from_moments(rewards: Sequence[float], mean: float, sample_std: float,
                            scale: ScaleRewards) -> list[float]:
    """Advantages of a local slice given moments of the *global* group (used for
    the distributed same-prompt reward scope)."""
    if ScaleRewards(scale) is ScaleRewards.NONE:
        return [float(r) - mean for r in rewards]
    return [(float(r) - mean) / (sample_std + GROUP_STD_EPS) for r in rewards]


def k3_kl(logp: float, logp_ref: float) -> float:
    d = logp_ref - logp
    return math.exp(d) - d - 1.0


def clipped_surrogate(ratio: float, advantage: float, eps_low: float, eps_high: float) -> float:
    unclipped = ratio * advantage
    clipped = min(max(ratio, 1.0 - eps_low), 1.0 + eps_high) * advantage
    return min(unclipped, clipped)


def tis_weight(logp_train: float, logp_rollout: float, cap: float) -> float:
    return min(math.exp(logp_train - logp_rollout), cap)


def sequence_log_ratio(logp: Sequence[float], logp_old: Sequence[float], mask: Sequence[float]) -> float:
    if not (len(logp) == len(logp_old) == len(mask)):
        raise ValueError("sequence_log_ratio: length mismatch")
    _check_mask(mask)
    denom = max(sum(mask), 1.0)
    num = sum((a - b) * m for a, b, m in zip(logp, logp_old, mask) if m > 0.0)
    return num / denom


def _check_mask(row: Sequence[float]) -> None:
    for m in row:
        if not (math.isfinite(m) and m >= 0.0):
            raise ValueError("masked_mean: mask entries must be finite and non-negative")


def _masked_total(values, mask) -> float:
    return sum(v * m for row, mrow in zip(values, mask) for v, m in zip(row, mrow) if m > 0.0)


def masked_mean(values: Sequence[Sequence[float]], mask: Sequence[Sequence[float]],
                loss_type: LossType = LossType.DAPO) -> float:
    if len(values) == 0:
        raise ValueError("masked_mean: empty batch")
    if len(values) != len(mask):
        raise ValueError("masked_mean: row count mismatch")
    width = len(values[0])
    if width == 0:
        raise ValueError("masked_mean: zero-width rows")
    for row, mrow in zip(values, mask):
        if len(row) != width or len(mrow) != width:
            raise ValueError("masked_mean: ragged row")
        _check_mask(mrow)
    loss_type = LossType(loss_type)
    if loss_type is LossType.GRPO:
        acc = 0.0
        for row, mrow in zip(values, mask):
            denom = max(sum(mrow), 1.0)
            acc += sum(v * m for v, m in zip(row, mrow) if m > 0.0) / denom
        return acc / len(values)
    if loss_type is LossType.DR_GRPO:
        return _masked_total(values, mask) / (len(values) * width)
    active = max(sum(sum(r) for r in mask), 1.0)
    return _masked_total(values, mask) / active


def zero_mask_rows(mask: Sequence[Sequence[float]]) -> int:
    return sum(1 for row in mask if sum(row) <= 0.0)


def grpo_loss_scalar(logp, logp_old, logp_ref, advantages, mask, *, eps_low, eps_high, beta,
                     loss_type=LossType.DAPO, is_level=ImportanceSamplingLevel.TOKEN,
                     dapo_norm: Optional[float] = None, tis_w=None) -> float:
    """Float64 list-of-lists restatement of the whole loss (test oracle)."""
    is_level = ImportanceSamplingLevel(is_level)
    loss_type = LossType(loss_type)
    per_token = []
    for g, (lp, lo, m) in enumerate(zip(logp, logp_old, mask)):
        if is_level is ImportanceSamplingLevel.SEQUENCE:
            s = min(max(sequence_log_ratio(lp, lo, m), -RATIO_LOG_CAP), RATIO_LOG_CAP)
            ratios = [math.exp(s)] * len(lp)
        else:
            ratios = [math.exp(min(max((a - b) if k > 0 else 0.0, -RATIO_LOG_CAP), RATIO_LOG_CAP))
                      for a, b, k in zip(lp, lo, m)]
        row = []
        for t, r in enumerate(ratios):
            a = advantages[g]
            v = 0.0 if a == 0.0 else clipped_surrogate(r, a, eps_low, eps_high)
            if tis_w is not None:
                v *= tis_w[g][t]
            if logp_ref is not None and m[t] > 0:
                v -= beta * k3_kl(lp[t], logp_ref[g][t])
            row.append(v)
        per_token.append(row)
    if loss_type is LossType.DAPO and dapo_norm is not None:
        return -_masked_total(per_token, mask) / max(dapo_norm, 1.0)
    return -masked_mean(per_token, mask, loss_type)


# --------------------------------------------------------------------------
# tensor loss
# --------------------------------------------------------------------------

@dataclass
class LossConfig:
    clip_eps_low: float = 0.2
    clip_eps_high: float = 0.2
    beta: float = 0.0
    loss_type: LossType = LossType.DAPO
    is_level: ImportanceSamplingLevel = ImportanceSamplingLevel.TOKEN
    dapo_norm: Optional[float] = None
    scale: float = 1.0  # extra multiplier (1/(accum*world) for non-DAPO reductions)


def grpo_loss_eager(logp: torch.Tensor, logp_old: torch.Tensor, logp_ref: Optional[torch.Tensor],
                    advantages: torch.Tensor, mask: torch.Tensor, cfg: LossConfig,
                    tis_w: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Eager PyTorch loss; shapes ``logp*``/``mask`` ``[G, L]``, ``advantages`` ``[G]`` or ``[G,1]``."""
    adv = advantages.reshape(-1, 1).to(logp.dtype)
    keep = mask > 0
    logp_r = torch.where(keep, logp, logp_old)  # padding contributes ratio exp(0), no gradient
    if ImportanceSamplingLevel(cfg.is_level) is ImportanceSamplingLevel.TOKEN:
        ratio = (logp_r - logp_old).clamp(-RATIO_LOG_CAP, RATIO_LOG_CAP).exp()
    else:
        lr = logp_r - logp_old
        denom = mask.sum(-1, keepdim=True).clamp(min=1.0)
        ratio = ((lr * mask).sum(-1, keepdim=True) / denom).clamp(-RATIO_LOG_CAP, RATIO_LOG_CAP).exp()
        ratio = ratio.expand_as(logp)
    unclipped = ratio * adv
    clipped = ratio.clamp(1.0 - cfg.clip_eps_low, 1.0 + cfg.clip_eps_high) * adv
    surrogate = torch.minimum(unclipped, clipped)
    surrogate = torch.where(adv.expand_as(surrogate) != 0, surrogate, torch.zeros_like(surrogate))
    if tis_w is not None:
        surrogate = surrogate * tis_w
    per_token = surrogate
    if logp_ref is not None:
        logp_kl = torch.where(keep, logp, logp_ref)
        d = logp_ref - logp_kl
        per_token = surrogate - cfg.beta * (d.exp() - d - 1.0)
    kept = torch.where(keep, per_token, torch.zeros_like(per_token)) * mask
    lt = LossType(cfg.loss_type)
    if lt is LossType.GRPO:
        red = (kept.sum(-1) / mask.sum(-1).clamp(min=1.0)).mean()
    elif lt is LossType.DR_GRPO:
        red = kept.sum() / float(mask.shape[0] * mask.shape[1])
    else:
        norm = max(cfg.dapo_norm, 1.0) if cfg.dapo_norm is not None else max(float(mask.sum()), 1.0)
        red = kept.sum() / norm
    return -red * cfg.scale


def grpo_loss(logp, logp_old, logp_ref, advantages, mask, cfg: LossConfig, tis_w=None) -> torch.Tensor:
    """Loss entry point used by the trainer: fused kernel on CUDA, eager on CPU."""
    from . import ops as _ops
    if _ops.native(logp):
        from .ops import grpo_loss_fused
        return grpo_loss_fused(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w)
    return grpo_loss_eager(logp, logp_old, logp_ref, advantages, mask, cfg, tis_w)


@dataclass
class LossStats:
    """Detached diagnostics of one loss evaluation (sums, so ranks can add them)."""

    kl_sum: float = 0.0
    clip_low_sum: float = 0.0
    clip_high_sum: float = 0.0
    token_count: float = 0.0


@torch.no_grad()
def loss_stats(logp, logp_old, logp_ref, advantages, mask, cfg: LossConfig) -> LossStats:
    keep = mask > 0
    adv = advantages.reshape(-1, 1)
    lr = torch.where(keep, logp - logp_old, torch.zeros_like(logp))
    if ImportanceSamplingLevel(cfg.is_level) is ImportanceSamplingLevel.SEQUENCE:
        lr = ((lr * mask).sum(-1, keepdim=True) / mask.sum(-1, keepdim=True).clamp(min=1.0)).expand_as(logp)
    ratio = lr.clamp(-RATIO_LOG_CAP, RATIO_LOG_CAP).exp()
    low = ((ratio < 1.0 - cfg.clip_eps_low) & (adv < 0) & keep).sum().item()
    high = ((ratio > 1.0 + cfg.clip_eps_high) & (adv > 0) & keep).sum().item()
    kl = 0.0
    if logp_ref is not None:
        d = torch.where(keep, logp_ref - logp, torch.zeros_like(logp))
        kl = float(((d.exp() - d - 1.0) * mask).sum().item())
    return LossStats(kl, float(low), float(high), float(mask.sum().item()))
