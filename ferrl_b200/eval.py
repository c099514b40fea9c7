"""Held-out evaluation: base policy (adapter off) versus adapted policy, avg@k.

Reference ``crates/ferrl/src/eval.rs:188-363``: for each held-out prompt sample
``group_size`` completions with the adapter disabled and again with it enabled,
on *paired* random substreams (the same global rows and draw indices for both
arms, so the comparison is not blurred by sampling noise), score them with the
task's reward function and report per-prompt and overall means.  The adapter
flag and the sampler state are restored on every exit path.  Evaluation samples
at ``EvalSampling`` (temperature 0.6, top-p 0.95 by default), not at the
training temperature.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field
from typing import Optional, Sequence

from .policy import EvalSampling, GenConfig, Policy
from .rewards import RewardFn, Sample

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
        if not math.isfinite(d):
            raise EvalError("adapter/base reward improvement must be finite")
        return d

    def to_json(self) -> dict:
        d = asdict(self)
        d["improvement"] = self.improvement()
        return d


def score_all(policy: Policy, reward_fn: RewardFn, tokenizer, samples: Sequence[Sample], gen: GenConfig,
              batch_prompts: int = 16) -> list[float]:
    """Mean reward per prompt under the policy's current adapter state."""
    means = []
    for s0 in range(0, len(samples), batch_prompts):
        chunk = samples[s0:s0 + batch_prompts]
        prompts = [list(tokenizer.encode(s.prompt)) for s in chunk]
        bases = [EVAL_ROW_BASE + (s0 + i) * gen.group_size for i in range(len(chunk))]
        rollouts = policy.generate_batch(prompts, gen, bases)
        for s, r in zip(chunk, rollouts):
            comps = [tokenizer.decode(r.completion(i)) for i in range(len(r))]
            rewards = reward_fn.reward_group(s, comps)
            if len(rewards) != len(comps):
                raise EvalError("reward function returned a different number of rewards than completions")
            means.append(sum(rewards) / len(rewards))
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
        policy.set_adapter_enabled(False)
        base = score_all(policy, reward_fn, tokenizer, samples, gen, batch_prompts)
        policy.set_adapter_enabled(True)
        adapted = score_all(policy, reward_fn, tokenizer, samples, gen, batch_prompts)
    finally:
        policy.set_adapter_enabled(prior)
        policy.restore_sampler_state(sampler_pre)
    return EvalReport(len(samples), gen.group_size, sum(base) / len(base), sum(adapted) / len(adapted),
                      [PromptEval(b, a) for b, a in zip(base, adapted)])
