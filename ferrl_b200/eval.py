"""Held-out evaluation: base policy (adapter off) versus adapted policy, avg@k.

Reference ``crates/ferrl/src/eval.rs:188-363``: for each held-out prompt sample
``group_size`` completions with the adapter disabled and again with it enabled,
on *paired* random substreams (the same global rows and draw indices for both
arms, so the comparison is not blurred by sampling noise), score them with the
task's reward function and report per-prompt and overall means.  The adapter
flag is restored on every exit path; the sampler keeps the progression of a
successful evaluation and is rolled back, and read back to prove it, when the
evaluation fails.  Rollouts and rewards are validated as the trainer validates
them (group size, prompt prefix, EOS semantics, one finite reward per
completion); means are order-independent compensated sums.  Evaluation samples
at ``EvalSampling`` (temperature 0.6, top-p 0.95 by default), not at the
training temperature.  Differences kept on purpose: the two arms run batch by
batch over all prompts (one adapter toggle per arm instead of two per prompt: a
toggle rebuilds the merged rollout weights), and eval rows live at
``EVAL_ROW_BASE`` so they never replay a training row's random stream.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Optional, Sequence

from .grpo import canonical_sum
from .policy import EvalSampling, GenConfig, Policy, RolloutSemanticsError, validate_generated_rollout_semantics
from .rewards import RewardError, RewardFn, Sample, validate_reward_values

EVAL_ROW_BASE = 1 << 40   # eval substreams live far away from any training row index


class EvalError(RuntimeError):
    pass


@dataclass
class PromptEval:
    base_mean: float
    adapter_mean: float


@dataclass
class EvalReport:
    n_prompts: int
    group_size: int
    base_reward_mean: float
    adapter_reward_mean: float
    per_prompt: list = field(default_factory=list)

    def improvement(self) -> float:
        d = self.adapter_reward_mean - self.base_reward_mean
        if not (math.isfinite(d) and _finite_f32(d)):
            raise EvalError(f"adapter/base reward improvement is outside finite f32: adapter={self.adapter_reward_mean:e}, "
                            f"base={self.base_reward_mean:e}")
        return d

    def to_json(self) -> dict:
        d = asdict(self)
        d["improvement"] = self.improvement()
        return d


def _finite_f32(x: float) -> bool:
    import struct
    try:
        return math.isfinite(struct.unpack("<f", struct.pack("<f", x))[0])
    except OverflowError:
        return False


def validated_mean(values: Sequence[float]) -> float:
    """Mean of finite values that does not depend on their order (compensated sum), eval.rs ``validated_mean``."""
    return canonical_sum([float(v) for v in values]) / len(values)


def score_all(policy: Policy, reward_fn: RewardFn, tokenizer, samples: Sequence[Sample], gen: GenConfig,
              batch_prompts: int = 16) -> list[float]:
    """Mean reward per prompt under the policy's current adapter state."""
    means = []
    for s0 in range(0, len(samples), batch_prompts):
        chunk = samples[s0:s0 + batch_prompts]
        prompts = [list(tokenizer.encode(s.prompt)) for s in chunk]
        for s, ids in zip(chunk, prompts):
            if not ids:
                raise EvalError(f"prompt encoded to zero tokens: {s.prompt!r}")
        bases = [EVAL_ROW_BASE + (s0 + i) * gen.group_size for i in range(len(chunk))]
        rollouts = policy.generate_batch(prompts, gen, bases)
        for s, ids, r in zip(chunk, prompts, rollouts):
            if len(r) != gen.group_size:
                raise EvalError(f"Policy::generate returned {len(r)} completions for group_size {gen.group_size}")
            if hasattr(r, "token_ids"):            # scripted doubles in tests carry rows only
                try:
                    validate_generated_rollout_semantics(r, ids, gen)
                except RolloutSemanticsError as e:
                    raise EvalError(str(e)) from e
            # only the real completion tokens reach the reward: EOS padding is never decoded
            comps = [tokenizer.decode(r.completion(i)) for i in range(len(r))]
            rewards = reward_fn.reward_group(s, comps)
            if len(rewards) != len(comps):
                raise EvalError(f"reward_group returned {len(rewards)} rewards for {len(comps)} completions")
            try:
                validate_reward_values(rewards)
            except RewardError as e:
                raise EvalError(str(e)) from e
            means.append(validated_mean(rewards))
    return means


def evaluate(policy: Policy, reward_fn: RewardFn, tokenizer, samples: Sequence[Sample], gen: GenConfig,
             batch_prompts: int = 16) -> EvalReport:
    if gen.group_size < 1:
        raise EvalError("group_size must be >= 1")
    if gen.max_new_tokens < 1:
        raise EvalError("max_new_tokens must be >= 1")
    if not samples:
        raise EvalError("no eval samples")
    if gen.eval_sampling is None:
        gen = GenConfig(gen.group_size, gen.max_new_tokens, gen.temperature, gen.eos_token_id, EvalSampling())
    sampler_pre = policy.sampler_state()
    prior = policy.adapter_enabled()
    try:
        try:
            policy.set_adapter_enabled(False)
            if policy.adapter_enabled():
                # full fine-tuning: the base weights are the trained weights, the comparison would be of the
                # policy against itself
                raise EvalError("the policy cannot disable its adapter (full fine-tuning mode?) — the base-vs-trained "
                                "comparison is unavailable; evaluate against a separately loaded base policy instead")
            base = score_all(policy, reward_fn, tokenizer, samples, gen, batch_prompts)
            policy.set_adapter_enabled(True)
            adapted = score_all(policy, reward_fn, tokenizer, samples, gen, batch_prompts)
            report = EvalReport(len(samples), gen.group_size, validated_mean(base), validated_mean(adapted),
                                [PromptEval(b, a) for b, a in zip(base, adapted)])
            report.improvement()            # refuse a report whose headline number cannot be formed
        finally:
            policy.set_adapter_enabled(prior)
    except BaseException as error:
        # a failed evaluation must not leave a partially advanced stochastic policy behind
        try:
            policy.restore_sampler_state(sampler_pre)
            exact = policy.sampler_state() == sampler_pre
        except Exception as rollback:  # noqa: BLE001
            raise EvalError(f"evaluation failed ({error}); exact sampler rollback also failed ({rollback}); "
                            "discard the policy instance") from error
        if not exact:
            raise EvalError(f"evaluation failed ({error}); the policy did not restore the exact pre-evaluation sampler "
                            "state; discard the policy instance") from error
        raise
    return report
