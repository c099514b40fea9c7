"""The policy seam: what the trainer needs from a language-model policy.

Mirrors the reference's ``trait Policy`` (``crates/ferrl/src/policy.rs:333-579``)
and ``Rollout``/``GenConfig``/``EvalSampling`` (``:25-63``, ``:248-305``): a
rollout of one prompt is ``group_size`` rows of ``prompt_len + max_new_tokens``
tokens, right-padded with EOS after each row's first EOS, with the number of
real completion tokens per row and the sampler's behaviour log-probs.

Difference from the reference: policies here are *batched*.  ``generate_batch``
takes several prompts at once (one decode batch of ``len(prompts)*group_size``
rows keeps a B200 busy; the reference decodes one group at a time), and
``token_logprobs`` scores a list of rollouts in one forward.  The single-prompt
methods are thin wrappers.
"""
from __future__ import annotations

from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch


@dataclass
class EvalSampling:
    temperature: float = 0.6
    top_p: Optional[float] = 0.95


@dataclass
class GenConfig:
    group_size: int = 8
    max_new_tokens: int = 256
    temperature: float = 1.0
    eos_token_id: Optional[int] = None
    eval_sampling: Optional[EvalSampling] = None
    top_p: Optional[float] = None  # training-time nucleus (None = full distribution)


@dataclass
class Rollout:
    token_ids: torch.Tensor            # int64 [G, prompt_len + max_new_tokens] (host)
    prompt_len: int
    completion_lens: list[int]
    rollout_logprobs: Optional[torch.Tensor] = None  # float32 [G, max_new_tokens]

    @staticmethod
    def rectangular(token_ids, prompt_len: int) -> "Rollout":
        t = torch.as_tensor(token_ids, dtype=torch.int64)
        return Rollout(t, prompt_len, [t.shape[1] - prompt_len] * t.shape[0], None)

    def __len__(self) -> int:
        return int(self.token_ids.shape[0])

    @property
    def width(self) -> int:
        return int(self.token_ids.shape[1]) - self.prompt_len

    def completion(self, row: int) -> list[int]:
        return self.token_ids[row, self.prompt_len:self.prompt_len + self.completion_lens[row]].tolist()


class RolloutSemanticsError(ValueError):
    pass


def validate_completion_semantics(completion: Sequence[int], real: int, eos: Optional[int]) -> None:
    n = len(completion)
    if real > n:
        raise RolloutSemanticsError(f"completion_len {real} exceeds generated width {n}")
    if eos is None:
        if real != n:
            raise RolloutSemanticsError(
                f"completion_len {real} is shortened without EOS; expected full generated width {n}")
        return
    first = next((i for i, t in enumerate(completion) if t == eos), None)
    expected = n if first is None else first + 1
    if real != expected:
        raise RolloutSemanticsError(
            f"completion_len {real} does not end immediately after the first EOS token; expected {expected}")
    if first is not None and any(t != eos for t in completion[expected:]):
        raise RolloutSemanticsError("completion contains a live non-EOS token after its first EOS")


def validate_generated_rollout_semantics(r: Rollout, prompt_ids: Sequence[int], gen: GenConfig) -> None:
    if r.prompt_len != len(prompt_ids):
        raise RolloutSemanticsError(
            f"rollout prompt_len {r.prompt_len} does not match encoded prompt length {len(prompt_ids)}")
    if len(r.completion_lens) != len(r):
        raise RolloutSemanticsError(f"rollout has {len(r.completion_lens)} completion_lens for {len(r)} rows")
    want = len(prompt_ids) + gen.max_new_tokens
    if r.token_ids.shape[1] != want:
        raise RolloutSemanticsError(f"rollout rows have length {r.token_ids.shape[1]}, expected {want}")
    p = torch.as_tensor(list(prompt_ids), dtype=torch.int64)
    if not bool((r.token_ids[:, :len(prompt_ids)] == p[None]).all()):
        raise RolloutSemanticsError("a rollout row prefix does not match the encoded prompt")
    # vectorised form of validate_completion_semantics over all rows
    comp = r.token_ids[:, len(prompt_ids):]
    lens = torch.as_tensor(r.completion_lens)
    N = comp.shape[1]
    if gen.eos_token_id is None:
        if not bool((lens == N).all()):
            raise RolloutSemanticsError("a completion is shortened without EOS")
    else:
        is_eos = comp == gen.eos_token_id
        first = torch.where(is_eos.any(1), is_eos.int().argmax(1) + 1, torch.full_like(lens, N))
        if not bool((first == lens).all()):
            row = int((first != lens).nonzero()[0])
            validate_completion_semantics(comp[row].tolist(), int(lens[row]), gen.eos_token_id)
        tail = torch.arange(N)[None, :] >= lens[:, None]
        if bool((tail & ~is_eos).any()):
            raise RolloutSemanticsError("completion contains a live non-EOS token after its first EOS")
    if r.rollout_logprobs is not None:
        live = torch.arange(N)[None, :] < lens[:, None]
        lp = r.rollout_logprobs[live]
        if not bool(torch.isfinite(lp).all()) or bool((lp > 0).any()):
            raise RolloutSemanticsError("behaviour log-probs must be finite and non-positive")


class Policy:
    """Abstract policy. Concrete: ``LmPolicy`` (any model family) and scripted
    fakes in the tests."""

    def generate_batch(self, prompts: Sequence[Sequence[int]], cfg: GenConfig,
                       global_row_bases: Sequence[int]) -> list[Rollout]:
        raise NotImplementedError

    def generate(self, prompt: Sequence[int], cfg: GenConfig, global_row_base: int = 0) -> Rollout:
        return self.generate_batch([prompt], cfg, [global_row_base])[0]

    def token_logprobs(self, rollouts: Sequence[Rollout]) -> torch.Tensor:
        """Grad-bearing ``[sum G, max_new_tokens]`` log-probs of the completions."""
        raise NotImplementedError

    def token_logprobs_detached(self, rollouts: Sequence[Rollout]) -> torch.Tensor:
        with torch.no_grad():
            return self.token_logprobs(rollouts)

    def backward(self, loss: torch.Tensor) -> None:
        loss.backward()

    def set_adapter_enabled(self, on: bool) -> None:
        raise NotImplementedError

    def adapter_enabled(self) -> bool:
        raise NotImplementedError

    def trainable_params(self) -> list[torch.nn.Parameter]:
        raise NotImplementedError

    def on_params_updated(self) -> None:
        """Called after each optimizer step (merged rollout weights go stale)."""

    def sampler_state(self) -> bytes:
        raise NotImplementedError

    def validate_sampler_state(self, state: bytes) -> None:
        raise NotImplementedError

    def restore_sampler_state(self, state: bytes) -> None:
        raise NotImplementedError

    def lora_recipe(self) -> Optional[str]:
        return None

    def device(self) -> torch.device:
        return torch.device("cpu")
