"""Reproducible GRPO sampler built on a counter RNG shared by host and device.

A row's random stream is a pure function of ``(base_seed, global_row_index)``
and the draw index within the row, so DP ranks, resumed runs and re-played
ledgers draw identical tokens no matter how rows are batched.  The reference
reaches the same contract by forking one Xoshiro256++ stream per row from a
SplitMix64-mixed seed (``crates/ferrl/src/sampler.rs:69-143``); here the whole
generator *is* the SplitMix64 finaliser applied to a counter, which a CUDA
thread can evaluate without carrying state.  The sm_100a sampling kernel
(``csrc/sample``) evaluates exactly ``uniform_u24`` below.

Sampling semantics (reference ``sampler.rs:228-297``): float32 softmax of
``logits / T``; optional nucleus filter that keeps the highest-probability
tokens until their mass reaches ``top_p`` (the crossing token included, ties
with it included too); the returned behaviour log-prob is the log of the kept,
renormalised probability of the drawn token.
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass
from typing import Optional

import torch

MASK64 = (1 << 64) - 1
GOLDEN = 0x9E3779B97F4A7C15


def splitmix64_finalize(z: int) -> int:
    z &= MASK64
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & MASK64
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & MASK64
    return z ^ (z >> 31)


def substream_key(base_seed: int, global_row: int) -> int:
    """Key of one row's stream (same mixing as reference sampler.rs:69-78)."""
    return splitmix64_finalize((base_seed + global_row * GOLDEN) & MASK64)


def uniform_u24(base_seed: int, global_row: int, draw: int) -> float:
    """Draw number ``draw`` of row ``global_row``: a multiple of 2^-24 in [0, 1),
    exactly representable in float32 so host and device agree bit for bit."""
    key = substream_key(base_seed, global_row)
    bits = splitmix64_finalize((key + (draw + 1) * GOLDEN) & MASK64)
    return (bits >> 40) * (1.0 / (1 << 24))


def _s64(c: int) -> int:
    c &= MASK64
    return c - (1 << 64) if c >= (1 << 63) else c


def _lsr(z: torch.Tensor, k: int) -> torch.Tensor:
    return (z >> k) & ((1 << (64 - k)) - 1)


def _mix_t(z: torch.Tensor) -> torch.Tensor:
    z = (z ^ _lsr(z, 30)) * _s64(0xBF58476D1CE4E5B9)
    z = (z ^ _lsr(z, 27)) * _s64(0x94D049BB133111EB)
    return z ^ _lsr(z, 31)


def uniforms_for_rows(base_seed: int, global_rows: torch.Tensor, draw: int) -> torch.Tensor:
    """Vectorised ``uniform_u24`` for int64 ``global_rows`` (two's-complement
    wrap-around multiplies reproduce the u64 arithmetic bit for bit)."""
    rows = global_rows.to(torch.int64)
    key = _mix_t(rows * _s64(GOLDEN) + _s64(base_seed))
    bits = _mix_t(key + _s64(((draw + 1) * GOLDEN) & MASK64))
    return (_lsr(bits, 40).to(torch.float32)) * (1.0 / (1 << 24))


def uniforms(base_seed: int, global_row_base: int, rows: int, draw: int) -> torch.Tensor:
    return uniforms_for_rows(base_seed, torch.arange(global_row_base, global_row_base + rows), draw)


def validate_top_p(top_p: Optional[float]) -> Optional[float]:
    if top_p is None:
        return None
    if not math.isfinite(top_p) or top_p <= 0.0 or top_p > 1.0:
        raise ValueError(f"top_p must be in (0, 1], got {top_p}")
    return None if top_p >= 1.0 else float(top_p)


def validate_temperature(t: float) -> float:
    if not math.isfinite(t) or t <= 0.0:
        raise ValueError(f"temperature must be finite and > 0, got {t}")
    return float(t)


def sample_from_logits_eager(logits: torch.Tensor, u: torch.Tensor, temperature: float,
                             top_p: Optional[float]) -> tuple[torch.Tensor, torch.Tensor]:
    """Reference sampler in plain PyTorch. ``logits`` ``[R, V]``, ``u`` ``[R]`` in [0,1).
    Returns ``(token int64 [R], behaviour_logprob float32 [R])``.  Tokens are
    drawn by inverse CDF in vocabulary order over the kept set."""
    temperature = validate_temperature(temperature)
    top_p = validate_top_p(top_p)
    probs = torch.softmax(logits.float() / temperature, dim=-1)
    if not torch.isfinite(probs).all():
        raise ValueError("sampler: non-finite probabilities")
    keep = torch.ones_like(probs, dtype=torch.bool)
    if top_p is not None:
        sp, _ = torch.sort(probs, dim=-1, descending=True)
        cum = sp.double().cumsum(-1)
        cross = (cum >= top_p).int().argmax(-1)  # first index reaching the mass
        never = ~(cum >= top_p).any(-1)
        thresh = sp.gather(-1, cross[:, None])
        thresh = torch.where(never[:, None], torch.zeros_like(thresh), thresh)
        keep = probs >= thresh
    kept = torch.where(keep, probs, torch.zeros_like(probs)).double()
    mass = kept.sum(-1)
    cdf = kept.cumsum(-1)
    target = u.double().to(logits.device) * mass
    tok = (cdf > target[:, None]).int().argmax(-1)
    # guard: u*mass rounding to the total picks the last kept token
    none = ~(cdf > target[:, None]).any(-1)
    if none.any():
        last = (kept > 0).int().flip(-1).argmax(-1)
        tok = torch.where(none, kept.shape[-1] - 1 - last, tok)
    lp = (kept.gather(-1, tok[:, None]).squeeze(-1) / mass).log().float()
    return tok.long(), lp


@dataclass
class GrpoSampler:
    """Sampler state: the run seed, the baked training temperature and nothing
    else - draws are addressed by (row, draw) counters supplied by the caller."""

    base_seed: int
    temperature: float = 1.0

    def __post_init__(self):
        self.base_seed = int(self.base_seed) & MASK64
        self.temperature = validate_temperature(self.temperature)

    def uniforms(self, global_row_base: int, rows: int, draw: int) -> torch.Tensor:
        return uniforms(self.base_seed, global_row_base, rows, draw)

    def sample(self, logits: torch.Tensor, global_rows, draw: int,
               temperature: Optional[float] = None, top_p: Optional[float] = None, draw_dev=None):
        """Sample one token per row of ``logits`` ``[R, V]``. ``global_rows`` is
        the first row's global index (rows are then consecutive) or an int64
        tensor ``[R]`` of global row indices."""
        t = self.temperature if temperature is None else validate_temperature(temperature)
        if isinstance(global_rows, int):
            global_rows = torch.arange(global_rows, global_rows + logits.shape[0])
        from . import ops as _ops
        if _ops.native(logits):
            from .ops import sample_top_p
            return sample_top_p(logits, self.base_seed, global_rows.to(logits.device), draw, t,
                                validate_top_p(top_p), draw_dev)
        u = uniforms_for_rows(self.base_seed, global_rows, draw)
        return sample_from_logits_eager(logits, u, t, top_p)

    # -- serialisable state (checkpoint manifest carries these bytes) --
    def state_bytes(self) -> bytes:
        return json.dumps({"kind": "counter-splitmix64", "version": 1, "base_seed": self.base_seed,
                           "temperature": self.temperature}, sort_keys=True).encode()

    @classmethod
    def from_state_bytes(cls, blob: bytes) -> "GrpoSampler":
        try:
            d = json.loads(blob.decode())
            if d.get("kind") != "counter-splitmix64" or d.get("version") != 1:
                raise ValueError("unknown sampler state kind/version")
            return cls(int(d["base_seed"]), float(d["temperature"]))
        except (KeyError, TypeError, json.JSONDecodeError, UnicodeDecodeError) as e:
            raise ValueError(f"malformed sampler state: {e}") from e

    def load_state_bytes(self, blob: bytes) -> None:
        other = self.from_state_bytes(blob)
        self.base_seed, self.temperature = other.base_seed, other.temperature
