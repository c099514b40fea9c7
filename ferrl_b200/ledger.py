"""Rollout ledger: persist collected rollouts so learning can happen later, elsewhere.

Reference ``crates/ferrl/src/rollout_ledger.rs`` (format v6 ``:19``): a window's
collection - prompt tokens, sampled tokens, completion lengths, behaviour
log-probs, rewards, advantages, loss masks, the controls it was collected under
(group size, width, reward scope, EOS, lr/beta of that step) and the sampler
state to hand to the next collector - is written as one step record under an
identity (trainer-config / policy / adapter / optimizer / sampler digests,
source step).  A reader refuses a ledger whose identity or controls differ
from the learner's expectations (``:1427-1890``).  Floats are stored as bit
patterns so a replay is bit-exact.

Layout: ``<dir>/manifest.json`` (format, identity, list of step files with
their SHA-256) and ``<dir>/step-<N>-rank<R>.json``.  Files are written to a
temp name, fsynced and renamed; the manifest is rewritten last.  Under data
parallelism every rank writes its own shard file and rank 0 commits the
manifest after all ranks report success.
"""
from __future__ import annotations

import hashlib
import json
import os
import struct
from dataclasses import asdict, dataclass, field
from typing import Optional, Sequence

import torch

from .policy import Rollout

LEDGER_FORMAT = 6
MANIFEST = "manifest.json"


class LedgerError(RuntimeError):
    pass


def f32_bits(x: float) -> int:
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


def bits_f32(b: int) -> float:
    return struct.unpack("<f", struct.pack("<I", int(b)))[0]


def f64_bits(x: float) -> int:
    return struct.unpack("<Q", struct.pack("<d", float(x)))[0]


def bits_f64(b: int) -> float:
    return struct.unpack("<d", struct.pack("<Q", int(b)))[0]


@dataclass
class LedgerIdentity:
    trainer_config_sha256: str
    policy_sha256: str
    adapter_sha256: str
    optimizer_sha256: str
    sampler_sha256: str
    source_step: int
    optimizer_step: int


@dataclass
class LedgerControls:
    grad_accum_steps: int
    prompts_per_item: int
    group_size: int
    completion_width: int
    reward_group_scope: str
    scale_rewards: str
    eos_token_id: Optional[int]
    truncation_masking: bool
    effective_lr_bits: int
    effective_beta_bits: int


@dataclass
class LedgerGroup:
    accum_index: int
    prompt_index: int
    rollout_global_row_base: int
    prompt_token_ids: list
    token_ids: list
    prompt_len: int
    completion_lens: list
    behavior_logprob_bits: Optional[list]
    reward_bits: list
    advantage_bits: list
    loss_mask: list

    @staticmethod
    def from_collected(accum_index: int, g) -> "LedgerGroup":
        r: Rollout = g.rollout
        lp = None if r.rollout_logprobs is None else \
            [[f32_bits(v) for v in row] for row in r.rollout_logprobs.tolist()]
        return LedgerGroup(accum_index, g.selection.prompt_index, g.selection.rollout_global_row_base,
                           list(g.prompt_ids), r.token_ids.tolist(), r.prompt_len, list(r.completion_lens), lp,
                           [f32_bits(x) for x in g.rewards], [f32_bits(x) for x in g.advantages],
                           [[int(v > 0) for v in row] for row in g.mask.tolist()])

    def rollout(self) -> Rollout:
        lp = None if self.behavior_logprob_bits is None else \
            torch.tensor([[bits_f32(b) for b in row] for row in self.behavior_logprob_bits], dtype=torch.float32)
        return Rollout(torch.tensor(self.token_ids, dtype=torch.int64), self.prompt_len, list(self.completion_lens), lp)

    def rewards(self) -> list:
        return [bits_f32(b) for b in self.reward_bits]

    def advantages(self) -> list:
        return [bits_f32(b) for b in self.advantage_bits]

    def mask(self) -> torch.Tensor:
        return torch.tensor(self.loss_mask, dtype=torch.float32)


@dataclass
class LedgerStep:
    step: int
    rank: int
    world_size: int
    controls: LedgerControls
    window_tokens: int
    live_items: int
    post_rollout_sampler_state: list
    groups: list = field(default_factory=list)

    def to_json(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_json(d: dict) -> "LedgerStep":
        try:
            c = LedgerControls(**d["controls"])
            groups = [LedgerGroup(**g) for g in d["groups"]]
            return LedgerStep(int(d["step"]), int(d["rank"]), int(d["world_size"]), c, int(d["window_tokens"]),
                              int(d["live_items"]), list(d["post_rollout_sampler_state"]), groups)
        except (KeyError, TypeError) as e:
            raise LedgerError(f"malformed ledger step: {e}") from e

    def validate(self) -> None:
        c = self.controls
        for g in self.groups:
            rows = len(g.token_ids)
            if rows != c.group_size:
                raise LedgerError(f"group at prompt {g.prompt_index} has {rows} rows, controls say {c.group_size}")
            if len(g.completion_lens) != rows or len(g.reward_bits) != rows or len(g.advantage_bits) != rows \
                    or len(g.loss_mask) != rows:
                raise LedgerError("per-row arrays of a ledger group disagree in length")
            width = g.prompt_len + c.completion_width
            for row, m, ln in zip(g.token_ids, g.loss_mask, g.completion_lens):
                if len(row) != width or len(m) != c.completion_width:
                    raise LedgerError("ledger row width does not match prompt_len + completion_width")
                if row[:g.prompt_len] != g.prompt_token_ids:
                    raise LedgerError("ledger row does not start with its prompt")
                if not 0 <= ln <= c.completion_width:
                    raise LedgerError("completion length out of range")
            if g.behavior_logprob_bits is not None:
                for row in g.behavior_logprob_bits:
                    for b in row:
                        v = bits_f32(b)
                        if v != v or v > 0:
                            raise LedgerError("behaviour log-probs must be finite and non-positive")


def _write_json_atomic(path: str, obj) -> str:
    tmp = path + ".tmp"
    data = json.dumps(obj, sort_keys=True).encode()
    with open(tmp, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())
    os.rename(tmp, path)
    return hashlib.sha256(data).hexdigest()


class RolloutLedgerWriter:
    def __init__(self, directory: str, identity: LedgerIdentity, *, rank: int = 0, world_size: int = 1):
        self.dir, self.identity, self.rank, self.world = directory, identity, rank, world_size
        os.makedirs(directory, exist_ok=True)
        self.entries: list = []
        mp = os.path.join(directory, MANIFEST)
        if os.path.exists(mp):
            man = json.load(open(mp))
            if man.get("identity") != asdict(identity):
                raise LedgerError("an existing ledger in this directory belongs to a different identity")
            self.entries = man.get("steps", [])

    def step_path(self, step: int, rank: int) -> str:
        return os.path.join(self.dir, f"step-{step:08d}-rank{rank}.json")

    def stage_step(self, st: LedgerStep) -> dict:
        """Write this rank's shard file; returns its manifest entry."""
        st.validate()
        if st.rank != self.rank or st.world_size != self.world:
            raise LedgerError("ledger step rank/world does not match the writer")
        p = self.step_path(st.step, st.rank)
        if os.path.exists(p):
            raise LedgerError(f"{p} already exists; ledger steps are never replaced")
        sha = _write_json_atomic(p, st.to_json())
        return {"step": st.step, "rank": st.rank, "file": os.path.basename(p), "sha256": sha}

    def commit(self, entries: Sequence[dict]) -> None:
        """Rank 0: publish the manifest covering ``entries`` (all ranks' shards of one step)."""
        self.entries = list(self.entries) + list(entries)
        _write_json_atomic(os.path.join(self.dir, MANIFEST),
                           {"format": LEDGER_FORMAT, "identity": asdict(self.identity), "world_size": self.world,
                            "steps": self.entries})

    def write_step(self, st: LedgerStep) -> None:
        """World-1 convenience: stage and commit."""
        self.commit([self.stage_step(st)])


class RolloutLedgerReader:
    def __init__(self, directory: str, expected: Optional[LedgerIdentity] = None, controls: Optional[LedgerControls] = None):
        self.dir = directory
        mp = os.path.join(directory, MANIFEST)
        try:
            man = json.load(open(mp))
        except (OSError, json.JSONDecodeError) as e:
            raise LedgerError(f"cannot read ledger manifest {mp}: {e}") from e
        if man.get("format") != LEDGER_FORMAT:
            raise LedgerError(f"unsupported ledger format {man.get('format')}")
        self.identity = LedgerIdentity(**man["identity"])
        if expected is not None and asdict(expected) != asdict(self.identity):
            diff = [k for k, v in asdict(expected).items() if asdict(self.identity).get(k) != v]
            raise LedgerError(f"ledger identity differs from the learner's expectation in {diff}")
        self.world = int(man.get("world_size", 1))
        self.entries = man["steps"]
        self.expected_controls = controls

    def steps(self) -> list:
        return sorted({e["step"] for e in self.entries})

    def read_step(self, step: int, rank: int = 0) -> LedgerStep:
        ent = next((e for e in self.entries if e["step"] == step and e["rank"] == rank), None)
        if ent is None:
            raise LedgerError(f"ledger has no shard for step {step} rank {rank}")
        p = os.path.join(self.dir, ent["file"])
        try:
            data = open(p, "rb").read()
        except OSError as e:
            raise LedgerError(f"cannot read {p}: {e}") from e
        if hashlib.sha256(data).hexdigest() != ent["sha256"]:
            raise LedgerError(f"{p} does not match its recorded SHA-256")
        st = LedgerStep.from_json(json.loads(data))
        st.validate()
        if self.expected_controls is not None:
            want, got = asdict(self.expected_controls), asdict(st.controls)
            bad = [k for k in want if k not in ("effective_lr_bits", "effective_beta_bits") and want[k] != got[k]]
            if bad:
                raise LedgerError(f"ledger controls differ from the learner's in {bad}")
        return st
