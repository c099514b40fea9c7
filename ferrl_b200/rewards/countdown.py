"""Countdown task: solvable-by-construction problem generator, prompt builder
and an exact-arithmetic tiered verifier.

Reference: ``crates/ferrl/src/countdown.rs`` - generator ``:470-611``
(SplitMix64, fold shuffled numbers with the first legal operator), prompt
``:132-150``, reward tiers ``:161-208`` (0 no answer tag; +0.1 well-formed
answer; +0.1 uses exactly the given numbers; +0.8 equals the target), exact
rational evaluator and ``expr := term (('+'|'-') term)*; term := factor
(('*'|'/') factor)*; factor := number | '(' expr ')'`` parser ``:256-466``.
Arithmetic is exact (``fractions.Fraction``); division by zero, unknown
characters, trailing tokens and numbers beyond u32 make the answer unparsable.
"""
from __future__ import annotations

from dataclasses import dataclass
from fractions import Fraction
from typing import Optional

from ..sampler import GOLDEN, MASK64, splitmix64_finalize

ANSWER_OPEN, ANSWER_CLOSE = "<answer>", "</answer>"
MAX_GEN_ATTEMPTS = 64

INSTRUCTIONS = ("Solve the countdown puzzle. Use each number exactly once with the operators + - * / and "
                "parentheses to write an arithmetic expression that equals the target. Give only the final "
                "expression between <answer> and </answer> tags.")
FEWSHOT = ("Numbers: 2, 3, 4\nTarget: 14\n<answer>2 * (3 + 4)</answer>\n\n"
           "Numbers: 5, 5, 2\nTarget: 12\n<answer>5 + 5 + 2</answer>\n")


@dataclass(frozen=True)
class CountdownProblem:
    numbers: tuple
    target: int

    @staticmethod
    def from_json(d) -> "CountdownProblem":
        return CountdownProblem(tuple(int(n) for n in d["numbers"]), int(d["target"]))

    def to_json(self):
        return {"numbers": list(self.numbers), "target": self.target}

    def split_key(self):
        """Identity of the problem for a train/eval split: the numbers as a multiset plus the target, so that a
        permutation of a training problem cannot land on the held-out side (crates/ferrl/src/countdown.rs:74-82)."""
        return tuple(sorted(self.numbers)), self.target

    def check(self, expression: str) -> bool:
        """Whether ``expression`` parses, uses every number exactly once and nothing else, and evaluates exactly
        to the target (crates/ferrl/src/countdown.rs:84-95)."""
        res = eval_expression(expression)
        if res is None:
            return False
        value, leaves = res
        return is_legal(leaves, self.numbers) and value.denominator == 1 and value.numerator == self.target


@dataclass(frozen=True)
class CountdownConfig:
    num_count: int = 3
    min_number: int = 1
    max_number: int = 20
    max_target: int = 1000


def build_prompt(p: CountdownProblem) -> str:
    nums = ", ".join(str(n) for n in p.numbers)
    return f"{INSTRUCTIONS}\n\n{FEWSHOT}\nNumbers: {nums}\nTarget: {p.target}\n"


class _Rng:
    def __init__(self, seed: int):
        self.s = seed & MASK64

    def next_u64(self) -> int:
        self.s = (self.s + GOLDEN) & MASK64
        return splitmix64_finalize(self.s)

    def range(self, a: int, b: int) -> int:
        lo, hi = min(a, b), max(a, b)
        return lo + self.next_u64() % (hi - lo + 1)

    def shuffled(self, items):
        v = list(items)
        for i in range(len(v) - 1, 0, -1):
            j = self.next_u64() % (i + 1)
            v[i], v[j] = v[j], v[i]
        return v


def _try_op(op: str, acc: int, x: int) -> Optional[int]:
    if op == "+":
        return acc + x
    if op == "*":
        return acc * x
    if op == "-":
        return acc - x if acc - x > 0 else None
    return acc // x if x != 0 and acc % x == 0 else None


def _build_one(rng: _Rng, cfg: CountdownConfig) -> CountdownProblem:
    numbers = [rng.range(cfg.min_number, cfg.max_number) for _ in range(max(cfg.num_count, 1))]
    order = rng.shuffled(numbers)
    acc = order[0]
    for x in order[1:]:
        for op in rng.shuffled(["+", "-", "*", "/"]):
            v = _try_op(op, acc, x)
            if v is not None:
                acc = v
                break
        else:
            acc = acc + x
    return CountdownProblem(tuple(numbers), acc)


def generate_dataset(seed: int, count: int, cfg: CountdownConfig = CountdownConfig()) -> list[CountdownProblem]:
    rng = _Rng(seed)
    out = []
    for _ in range(count):
        prob = None
        for _ in range(MAX_GEN_ATTEMPTS):
            prob = _build_one(rng, cfg)
            if 1 <= prob.target <= cfg.max_target:
                break
        else:
            prob = _build_one(rng, cfg)
        out.append(prob)
    return out


# ------------------------------------------------------------- verifier
def extract_answer(text: str) -> Optional[str]:
    i = text.find(ANSWER_OPEN)
    if i < 0:
        return None
    after = text[i + len(ANSWER_OPEN):]
    j = after.find(ANSWER_CLOSE)
    if j < 0:
        return None
    return after[:j].strip()


def _tokenize(s: str):
    toks = []
    i = 0
    while i < len(s):
        c = s[i]
        if c in "0123456789":
            j = i
            while j < len(s) and s[j] in "0123456789":
                j += 1
            v = int(s[i:j])
            if v > 0xFFFFFFFF:
                return None
            toks.append(v)
            i = j
        elif c in "+-*/()":
            toks.append(c)
            i += 1
        elif c in " \t\n\r":
            i += 1
        else:
            return None
    return toks


class _Parser:
    def __init__(self, toks):
        self.toks, self.pos, self.leaves = toks, 0, []

    def peek(self):
        return self.toks[self.pos] if self.pos < len(self.toks) else None

    def expr(self):
        acc = self.term()
        while acc is not None and self.peek() in ("+", "-"):
            op = self.toks[self.pos]
            self.pos += 1
            rhs = self.term()
            if rhs is None:
                return None
            acc = acc + rhs if op == "+" else acc - rhs
        return acc

    def term(self):
        acc = self.factor()
        while acc is not None and self.peek() in ("*", "/"):
            op = self.toks[self.pos]
            self.pos += 1
            rhs = self.factor()
            if rhs is None:
                return None
            if op == "*":
                acc = acc * rhs
            else:
                if rhs == 0:
                    return None
                acc = acc / rhs
        return acc

    def factor(self):
        t = self.peek()
        if t is None:
            return None
        self.pos += 1
        if isinstance(t, int):
            self.leaves.append(t)
            return Fraction(t)
        if t == "(":
            v = self.expr()
            if v is None or self.peek() != ")":
                return None
            self.pos += 1
            return v
        return None


def is_legal(leaves, numbers) -> bool:
    """The expression's leaves are the problem's numbers as a multiset."""
    return sorted(leaves) == sorted(numbers)


def eval_expression(s: str):
    """``(value, leaves)`` or ``None`` when the text is not a well-formed expression."""
    toks = _tokenize(s)
    if not toks:
        return None
    p = _Parser(toks)
    v = p.expr()
    if v is None or p.pos != len(toks):
        return None
    return v, p.leaves


@dataclass
class CountdownReward:
    format_reward: float = 0.1
    legal_reward: float = 0.1
    correct_reward: float = 0.8

    def score(self, problem: CountdownProblem, completion: str) -> float:
        ans = extract_answer(completion)
        if ans is None:
            return 0.0
        reward = self.format_reward
        res = eval_expression(ans)
        if res is None:
            return reward
        value, leaves = res
        if is_legal(leaves, problem.numbers):
            reward += self.legal_reward
            if value.denominator == 1 and value.numerator == problem.target:
                reward += self.correct_reward
        return reward

    # RewardFn surface (duck-typed; see rewards.RewardFn)
    def reward(self, sample, completion: str) -> float:
        return self.score(sample.target, completion)

    def reward_group(self, sample, completions):
        return [self.reward(sample, c) for c in completions]

    def reward_group_detailed(self, sample, completions):
        from . import RewardOutcome
        return [RewardOutcome(r) for r in self.reward_group(sample, completions)]
