"""Math task: exact-match ``<answer>`` reward after whitespace/comma
normalisation (reference ``crates/ferrl/src/math.rs:88-143``)."""
from __future__ import annotations

from dataclasses import dataclass

from .countdown import extract_answer


@dataclass(frozen=True)
class MathProblem:
    answer: str

    @staticmethod
    def from_json(d) -> "MathProblem":
        if not isinstance(d, dict) or not isinstance(d.get("answer"), str):
            raise ValueError("math target needs a string 'answer'")
        return MathProblem(d["answer"])

    def to_json(self):
        return {"answer": self.answer}


def math_split_key(sample):
    """Identity of a sample for a train/eval split: prompt and answer with ASCII whitespace and thousands separators
    removed, so that ``1, 000 + 234`` and ``1000 + 234`` cannot sit on both sides (crates/ferrl/src/math.rs:55-62)."""
    return normalize(sample.prompt), normalize(sample.target.answer)


def math_prompt(question: str) -> str:
    return f"{question}\nPut your final answer inside <answer></answer> tags.\n"


def normalize(s: str) -> str:
    # space, tab, line feed, form feed, carriage return (Rust's ``is_ascii_whitespace``: no vertical tab) and ','
    return "".join(c for c in s if c not in " \t\n\x0c\r,")


@dataclass
class MathReward:
    correct_reward: float = 1.0

    def score(self, expected: str, completion: str) -> float:
        got = extract_answer(completion)
        return self.correct_reward if got is not None and normalize(got) == normalize(expected) else 0.0

    def reward(self, sample, completion: str) -> float:
        return self.score(sample.target.answer, completion)

    def reward_group(self, sample, completions):
        return [self.reward(sample, c) for c in completions]

    def reward_group_detailed(self, sample, completions):
        from . import RewardOutcome
        return [RewardOutcome(r) for r in self.reward_group(sample, completions)]
