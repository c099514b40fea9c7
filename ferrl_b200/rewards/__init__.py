"""Typed-task reward verifiers: the ``RewardFn`` seam, ``Sample`` records, JSONL
data loading and deterministic train/eval splits.

Reference: ``crates/ferrl/src/reward.rs:80-178`` (``RewardFn`` with per-item,
per-group and detailed-group forms), ``sample.rs:38-43``, ``data.rs:59-230``.
"""
from __future__ import annotations

import json
import math as _math
from dataclasses import dataclass
from typing import Any, Callable, Generic, Hashable, Optional, Sequence, TypeVar

T = TypeVar("T")


class RewardError(RuntimeError):
    pass


class DataError(ValueError):
    pass


@dataclass(frozen=True)
class Sample(Generic[T]):
    prompt: str
    target: Any

    def key(self) -> str:
        return json.dumps({"prompt": self.prompt, "target": _plain(self.target)}, sort_keys=True)


def _plain(x):
    if hasattr(x, "to_json"):
        return x.to_json()
    if hasattr(x, "__dict__") and not isinstance(x, dict):
        return {k: _plain(v) for k, v in vars(x).items()}
    if isinstance(x, (list, tuple)):
        return [_plain(v) for v in x]
    return x


@dataclass
class RewardOutcome:
    reward: float
    diagnostic: Optional[str] = None
    metadata: Optional[dict] = None


def validate_reward_values(rewards: Sequence[float]) -> None:
    for r in rewards:
        if not _math.isfinite(r):
            raise RewardError(f"reward function returned a non-finite reward {r!r}")


class RewardFn:
    """Override ``reward``; ``reward_group`` / ``reward_group_detailed`` default to
    mapping it over the group (a verifier that amortises per-group work, e.g. the
    sandboxed TriMul verifier, overrides the group forms)."""

    def reward(self, sample: Sample, completion: str) -> float:
        raise NotImplementedError

    def reward_group(self, sample: Sample, completions: Sequence[str]) -> list[float]:
        out = [float(self.reward(sample, c)) for c in completions]
        validate_reward_values(out)
        return out

    def reward_group_detailed(self, sample: Sample, completions: Sequence[str]) -> list[RewardOutcome]:
        rewards = self.reward_group(sample, completions)
        validate_reward_values(rewards)
        return [RewardOutcome(r) for r in rewards]


class FnReward(RewardFn):
    """Adapter: a plain ``(sample, completion) -> float`` callable as a ``RewardFn``."""

    def __init__(self, fn: Callable[[Sample, str], float]):
        self.fn = fn

    def reward(self, sample, completion):
        return self.fn(sample, completion)


# ------------------------------------------------------------------ data
def parse_jsonl(text: str, target_from_json: Callable[[Any], Any] = lambda x: x) -> list[Sample]:
    out = []
    for i, line in enumerate(text.splitlines()):
        if not line.strip():
            continue
        try:
            d = json.loads(line)
            if not isinstance(d, dict) or set(d.keys()) != {"prompt", "target"} or not isinstance(d["prompt"], str):
                raise ValueError("expected an object with exactly 'prompt' (string) and 'target'")
            out.append(Sample(d["prompt"], target_from_json(d["target"])))
        except (ValueError, KeyError, TypeError) as e:
            raise DataError(f"line {i + 1}: {e}") from e
    return out


def read_jsonl(path: str, target_from_json: Callable[[Any], Any] = lambda x: x) -> list[Sample]:
    try:
        with open(path, encoding="utf-8") as f:
            return parse_jsonl(f.read(), target_from_json)
    except OSError as e:
        raise DataError(f"cannot read {path}: {e}") from e


class _SplitMix:
    def __init__(self, seed: int):
        self.s = seed & ((1 << 64) - 1)

    def next_u64(self) -> int:
        from ..sampler import GOLDEN, MASK64, splitmix64_finalize
        self.s = (self.s + GOLDEN) & MASK64
        return splitmix64_finalize(self.s)


def _shuffle(items: list, seed: int) -> None:
    rng = _SplitMix(seed)
    for i in range(len(items) - 1, 0, -1):
        j = rng.next_u64() % (i + 1)
        items[i], items[j] = items[j], items[i]


def train_eval_split(samples: Sequence[Sample], eval_n: int, seed: int):
    """Deduplicate (first seen wins), seeded Fisher-Yates shuffle, hold out the
    last ``eval_n`` (reference data.rs:145-182)."""
    seen, unique = set(), []
    for s in samples:
        k = s.key()
        if k not in seen:
            seen.add(k)
            unique.append(s)
    _shuffle(unique, seed)
    n = min(eval_n, len(unique))
    return unique[:len(unique) - n], unique[len(unique) - n:]


def train_eval_split_by_key(samples: Sequence[Sample], eval_n: int, seed: int,
                            key: Callable[[Sample], Hashable]):
    """Split whole key-groups so no key appears on both sides (reference
    data.rs:185-230): shuffle groups, hold out trailing groups until at least
    ``eval_n`` rows are held out."""
    groups: list[list[Sample]] = []
    pos: dict = {}
    for s in samples:
        k = key(s)
        if k in pos:
            groups[pos[k]].append(s)
        else:
            pos[k] = len(groups)
            groups.append([s])
    _shuffle(groups, seed)
    target = min(eval_n, sum(len(g) for g in groups))
    held, n_groups = 0, 0
    for g in reversed(groups):
        if held >= target:
            break
        held += len(g)
        n_groups += 1
    split = len(groups) - n_groups
    train = [s for g in groups[:split] for s in g]
    ev = [s for g in groups[split:] for s in g]
    return train, ev


from .countdown import CountdownConfig, CountdownProblem, CountdownReward, build_prompt, generate_dataset  # noqa: E402,F401
from .math import MathProblem, MathReward, math_prompt  # noqa: E402,F401
