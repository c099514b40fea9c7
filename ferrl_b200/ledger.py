"""Rollout ledger: persist collected rollouts so learning can happen later, elsewhere.

Reference ``crates/ferrl/src/rollout_ledger.rs`` (format v6 ``:19``): a window's
collection - prompt tokens, sampled tokens, completion lengths, behaviour
log-probs, rewards, advantages, loss masks, the controls it was collected under
(group size, width, reward scope, EOS, TIS cap, lr/beta of that step) and the
sampler state to hand to the next collector - is one published artifact under an
identity (trainer-config / policy / tensor-schema / adapter / optimizer / sampler
/ lineage digests, source step).  A reader refuses a window whose identity or
controls differ from the learner's expectations (``:1427-1890``).  Floats are
stored as bit patterns so a replay is bit-exact.

Layout (file names as in the reference, ``:21-24``, ``:1903``, ``:1985``)::

    <root>/step-<step:020>/window.json                 one-rank payload
    <root>/step-<step:020>/rank-<rank:05>.window.json  one payload per rank (distributed)
    <root>/step-<step:020>/.ferrl-ledger-owner         who staged a distributed window
    <root>/step-<step:020>/manifest.json               commit marker, linked last

A window is staged in a hidden sibling directory (``.tmp-step-...``): payloads
are created exclusively and fsynced, the manifest (identity, payload names,
lengths and SHA-256; for a distributed window also world size, controls and the
window totals) is written last.  Publication claims the final directory with
``mkdir`` - an existing window is never replaced - hard-links the payloads and
then the manifest, and syncs the directories.  A reader treats a directory
without ``manifest.json`` as absent.  Under data parallelism rank 0 creates the
stage, every rank writes its shard into it, and rank 0 commits once all ranks
report success or removes the stage when any rank failed (``:676-1110``).
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
PAYLOAD = "window.json"
OWNER_FILE = ".ferrl-ledger-owner"
DISTRIBUTED_KIND = "distributed_rollout_ledger"
_ZERO_DIGEST = "0" * 64


def step_dir_name(step: int) -> str:
    return f"step-{step:020d}"


def shard_payload_name(rank: int) -> str:
    return f"rank-{rank:05d}.window.json"


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
    tensor_schema_sha256: str = _ZERO_DIGEST
    lineage_sha256: str = _ZERO_DIGEST

    def validate(self) -> None:
        for k, v in asdict(self).items():
            if k.endswith("_sha256"):
                if not (isinstance(v, str) and len(v) == 64 and all(c in "0123456789abcdef" for c in v)):
                    raise LedgerError(f"ledger identity field {k} is not a lowercase SHA-256 hex digest")
        if self.source_step < 0 or self.optimizer_step < 0:
            raise LedgerError("ledger identity steps must be non-negative")


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
    tis_imp_ratio_cap_bits: Optional[int] = None


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




# ------------------------------------------------------------------ durable file helpers
def _write_new_synced(path: str, data: bytes) -> None:
    """Create ``path`` exclusively (never overwrite), write and fsync."""
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
    try:
        with os.fdopen(fd, "wb") as f:
            f.write(data)
            f.flush()
            os.fsync(f.fileno())
    except BaseException:
        try:
            os.unlink(path)
        except OSError:
            pass
        raise


def _sync_dir(path: str) -> None:
    fd = os.open(path or ".", os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def _remove_tree(path: str) -> None:
    """Remove a staging directory created by this module (flat: files only)."""
    try:
        for name in os.listdir(path):
            os.unlink(os.path.join(path, name))
        os.rmdir(path)
    except FileNotFoundError:
        pass


def _payload_bytes(st: "LedgerStep") -> bytes:
    return json.dumps(st.to_json(), sort_keys=True).encode()


def _entry(name: str, data: bytes, rank: Optional[int] = None) -> dict:
    e = {"payload_file": name, "payload_len": len(data), "payload_sha256": hashlib.sha256(data).hexdigest()}
    if rank is not None:
        e = {"rank": rank, **e}
    return e


@dataclass
class DistributedStage:
    """A hidden staging directory of one distributed window (created by rank 0)."""
    path: str
    final_dir: str
    owner: bytes
    step: int
    world_size: int


class RolloutLedgerWriter:
    """Writer bound to one learner pre-state identity (one window: ``identity.source_step``)."""

    def __init__(self, directory: str, identity: LedgerIdentity, *, rank: int = 0, world_size: int = 1,
                 fault_hook=None):
        identity.validate()
        self.dir, self.identity, self.rank, self.world = directory, identity, rank, world_size
        self.fault_hook = fault_hook            # tests: called with a stage name before each publication stage
        os.makedirs(directory, exist_ok=True)

    # -- paths
    def step_dir(self, step: int) -> str:
        return os.path.join(self.dir, step_dir_name(step))

    def step_path(self, step: int, rank: int) -> str:
        name = PAYLOAD if self.world == 1 else shard_payload_name(rank)
        return os.path.join(self.step_dir(step), name)

    def stage_path(self, step: int, nonce: int) -> str:
        kind = "distributed" if self.world > 1 else "local"
        return os.path.join(self.dir, f".tmp-{step_dir_name(step)}-{kind}-{nonce & (2 ** 64 - 1):016x}")

    def _fault(self, where: str) -> None:
        if self.fault_hook is not None:
            self.fault_hook(where)

    def _check_step(self, st: LedgerStep) -> None:
        st.validate()
        if st.step != self.identity.source_step:
            raise LedgerError(f"payload step {st.step} does not match identity source_step {self.identity.source_step}")
        if os.path.exists(os.path.join(self.step_dir(st.step), MANIFEST)):
            raise LedgerError(f"{self.step_dir(st.step)} already exists; ledger windows are never replaced")

    def _publish(self, stage: str, final_dir: str, names: Sequence[str]) -> None:
        """Claim ``final_dir``, link payloads, link the manifest last, sync."""
        try:
            os.mkdir(final_dir)                                   # atomic claim
        except FileExistsError:
            if os.path.exists(os.path.join(final_dir, MANIFEST)):
                raise LedgerError(f"{final_dir} already exists; ledger windows are never replaced") from None
            raise LedgerError(f"{final_dir} exists without a manifest (an interrupted or concurrent publication); "
                              "it is not reader-visible and must be removed before this window can be written") from None
        try:
            for name in names:
                os.link(os.path.join(stage, name), os.path.join(final_dir, name))
            self._fault("before_manifest_link")
            _sync_dir(final_dir)
            os.link(os.path.join(stage, MANIFEST), os.path.join(final_dir, MANIFEST))
        except BaseException:
            _remove_tree(final_dir)                               # nothing reader-visible was committed
            raise
        _sync_dir(final_dir)
        _sync_dir(self.dir)
        _remove_tree(stage)
        _sync_dir(self.dir)

    # -- one rank
    def write_step(self, st: LedgerStep) -> str:
        """Stage and publish a complete one-rank window; returns the window directory."""
        if self.world != 1 or st.world_size != 1 or st.rank != 0:
            raise LedgerError("write_step publishes one-rank windows; use the distributed stage for more ranks")
        self._check_step(st)
        stage = self.stage_path(st.step, int.from_bytes(os.urandom(8), "little"))
        os.mkdir(stage)
        try:
            data = _payload_bytes(st)
            _write_new_synced(os.path.join(stage, PAYLOAD), data)
            man = {"format_version": LEDGER_FORMAT, "identity": asdict(self.identity), **_entry(PAYLOAD, data)}
            _write_new_synced(os.path.join(stage, MANIFEST), json.dumps(man, sort_keys=True).encode())
            _sync_dir(stage)
            self._publish(stage, self.step_dir(st.step), [PAYLOAD])
        except BaseException:
            _remove_tree(stage)
            raise
        return self.step_dir(st.step)

    # -- several ranks
    def create_distributed_stage(self, step: int, nonce: int) -> DistributedStage:
        """Rank 0: make the hidden stage all ranks write their shard into."""
        if self.world <= 1:
            raise LedgerError("distributed ledger staging requires world_size > 1")
        if step != self.identity.source_step:
            raise LedgerError(f"distributed stage step {step} does not match identity source_step "
                              f"{self.identity.source_step}")
        if os.path.exists(os.path.join(self.step_dir(step), MANIFEST)):
            raise LedgerError(f"{self.step_dir(step)} already exists; ledger windows are never replaced")
        path = self.stage_path(step, nonce)
        os.mkdir(path)
        owner = f"{os.getpid()}:{nonce & (2 ** 64 - 1):016x}".encode()
        _write_new_synced(os.path.join(path, OWNER_FILE), owner)
        _sync_dir(path)
        _sync_dir(self.dir)
        return DistributedStage(path, self.step_dir(step), owner, step, self.world)

    def open_distributed_stage(self, step: int, nonce: int) -> DistributedStage:
        """Other ranks: the stage rank 0 created under the agreed nonce."""
        path = self.stage_path(step, nonce)
        try:
            owner = open(os.path.join(path, OWNER_FILE), "rb").read()
        except OSError as e:
            raise LedgerError(f"distributed stage {path} is not visible on this rank: {e}") from e
        return DistributedStage(path, self.step_dir(step), owner, step, self.world)

    def write_distributed_shard(self, stage: DistributedStage, st: LedgerStep) -> dict:
        """Write and sync this rank's immutable payload into ``stage``; returns its manifest entry."""
        st.validate()
        if st.world_size != self.world or st.rank != self.rank or not 0 <= st.rank < st.world_size:
            raise LedgerError(f"distributed shard has invalid rank {st.rank}/world {st.world_size} for this writer")
        if st.step != stage.step:
            raise LedgerError(f"payload step {st.step} does not match the stage's step {stage.step}")
        data = _payload_bytes(st)
        self._fault("before_shard_write")
        _write_new_synced(os.path.join(stage.path, shard_payload_name(st.rank)), data)
        return _entry(shard_payload_name(st.rank), data, rank=st.rank)

    def abort_distributed_stage(self, stage: DistributedStage) -> None:
        """Rank 0, after every rank reported that it stopped writing: drop the uncommitted stage."""
        try:
            owner = open(os.path.join(stage.path, OWNER_FILE), "rb").read()
        except FileNotFoundError:
            return
        if owner != stage.owner:
            raise LedgerError(f"stage {stage.path} changed owner; refusing to remove it")
        _remove_tree(stage.path)
        _sync_dir(self.dir)

    def commit_distributed_stage(self, stage: DistributedStage) -> str:
        """Rank 0: validate the shards against one another, write the manifest and publish."""
        shards, steps = [], []
        for r in range(stage.world_size):
            p = os.path.join(stage.path, shard_payload_name(r))
            try:
                data = open(p, "rb").read()
            except OSError as e:
                raise LedgerError(f"distributed stage is missing the shard of rank {r}: {e}") from e
            st = LedgerStep.from_json(json.loads(data))
            st.validate()
            if st.rank != r or st.world_size != stage.world_size or st.step != stage.step:
                raise LedgerError(f"shard {p} declares rank {st.rank}/world {st.world_size}/step {st.step}")
            shards.append(_entry(shard_payload_name(r), data, rank=r))
            steps.append(st)
        first = asdict(steps[0].controls)
        for st in steps[1:]:
            if asdict(st.controls) != first:
                raise LedgerError(f"rank {st.rank} collected under different controls than rank 0")
        seen: set = set()
        for st in steps:
            for g in st.groups:
                key = (g.accum_index, g.rollout_global_row_base)
                if key in seen:
                    raise LedgerError(f"two shards claim rollout rows starting at {g.rollout_global_row_base}")
                seen.add(key)
        man = {"format_version": LEDGER_FORMAT, "kind": DISTRIBUTED_KIND, "identity": asdict(self.identity),
               "step": stage.step, "world_size": stage.world_size, "controls": first,
               "window_tokens": sum(st.window_tokens for st in steps),
               "live_items": sum(st.live_items for st in steps), "shards": shards}
        _write_new_synced(os.path.join(stage.path, MANIFEST), json.dumps(man, sort_keys=True).encode())
        _sync_dir(stage.path)
        self._publish(stage.path, stage.final_dir, [OWNER_FILE] + [s["payload_file"] for s in shards])
        return stage.final_dir


class RolloutLedgerReader:
    def __init__(self, directory: str, expected: Optional[LedgerIdentity] = None, controls: Optional[LedgerControls] = None):
        self.dir = directory
        if not os.path.isdir(directory):
            raise LedgerError(f"ledger root {directory} does not exist")
        self.expected = expected
        self.expected_controls = controls

    def steps(self) -> list:
        """Published windows (directories that carry their commit marker)."""
        out = []
        for name in os.listdir(self.dir):
            if name.startswith("step-") and os.path.isfile(os.path.join(self.dir, name, MANIFEST)):
                try:
                    out.append(int(name[5:]))
                except ValueError:
                    continue
        return sorted(out)

    def _manifest(self, step: int) -> tuple:
        d = os.path.join(self.dir, step_dir_name(step))
        mp = os.path.join(d, MANIFEST)
        try:
            man = json.load(open(mp))
        except FileNotFoundError:
            raise LedgerError(f"ledger has no published window for step {step}") from None
        except (OSError, json.JSONDecodeError) as e:
            raise LedgerError(f"cannot read ledger manifest {mp}: {e}") from e
        if man.get("format_version") != LEDGER_FORMAT:
            raise LedgerError(f"unsupported ledger format {man.get('format_version')}")
        try:
            ident = LedgerIdentity(**man["identity"])
        except (KeyError, TypeError) as e:
            raise LedgerError(f"malformed ledger identity in {mp}: {e}") from e
        if self.expected is not None and asdict(self.expected) != asdict(ident):
            diff = [k for k, v in asdict(self.expected).items() if asdict(ident).get(k) != v]
            raise LedgerError(f"ledger identity differs from the learner's expectation in {diff}")
        if ident.source_step != step:
            raise LedgerError(f"window in {d} was collected for step {ident.source_step}")
        return d, man, ident

    def identity(self, step: int) -> LedgerIdentity:
        return self._manifest(step)[2]

    def consumed_ledger_sha256(self, step: int) -> str:
        """SHA-256 of the window's commit marker (which itself records every payload's digest): the
        value a learner binds into its continuation as "the ledger I consumed"."""
        self._manifest(step)
        return hashlib.sha256(open(os.path.join(self.dir, step_dir_name(step), MANIFEST), "rb").read()).hexdigest()

    def _payload(self, d: str, ent: dict) -> "LedgerStep":
        p = os.path.join(d, ent["payload_file"])
        try:
            data = open(p, "rb").read()
        except OSError as e:
            raise LedgerError(f"cannot read {p}: {e}") from e
        if len(data) != ent["payload_len"] or hashlib.sha256(data).hexdigest() != ent["payload_sha256"]:
            raise LedgerError(f"{p} does not match its recorded length and SHA-256")
        try:
            st = LedgerStep.from_json(json.loads(data))
        except json.JSONDecodeError as e:
            raise LedgerError(f"{p} is not valid JSON: {e}") from e
        st.validate()
        if self.expected_controls is not None:
            want, got = asdict(self.expected_controls), asdict(st.controls)
            bad = [k for k in want if k not in ("effective_lr_bits", "effective_beta_bits") and want[k] != got[k]]
            if bad:
                raise LedgerError(f"ledger controls differ from the learner's in {bad}")
        return st

    def world_size(self, step: int) -> int:
        man = self._manifest(step)[1]
        return int(man["world_size"]) if man.get("kind") == DISTRIBUTED_KIND else 1

    def read_step(self, step: int, rank: int = 0) -> LedgerStep:
        """The window of ``step`` (one-rank ledger) or ``rank``'s shard of it (distributed ledger)."""
        d, man, _ = self._manifest(step)
        if man.get("kind") == DISTRIBUTED_KIND:
            ent = next((e for e in man["shards"] if e["rank"] == rank), None)
            if ent is None:
                raise LedgerError(f"ledger has no shard for step {step} rank {rank}")
            st = self._payload(d, ent)
            if st.rank != rank or st.world_size != man["world_size"] or st.step != step:
                raise LedgerError(f"shard of rank {rank} declares rank {st.rank}/world {st.world_size}/step {st.step}")
            if asdict(st.controls) != man["controls"]:
                raise LedgerError(f"shard of rank {rank} disagrees with the manifest's controls")
            return st
        if rank != 0:
            raise LedgerError(f"ledger has no shard for step {step} rank {rank}")
        st = self._payload(d, man)
        if st.step != step or st.world_size != 1:
            raise LedgerError(f"window in {d} declares step {st.step}/world {st.world_size}")
        return st

    def read_distributed_step(self, step: int) -> list:
        """Every rank's shard of a distributed window, in rank order, with the totals checked."""
        d, man, _ = self._manifest(step)
        if man.get("kind") != DISTRIBUTED_KIND:
            raise LedgerError(f"window of step {step} is not a distributed ledger")
        ranks = sorted(e["rank"] for e in man["shards"])
        if ranks != list(range(int(man["world_size"]))):
            raise LedgerError(f"distributed manifest lists ranks {ranks} for world {man['world_size']}")
        shards = [self.read_step(step, r) for r in ranks]
        if sum(s.window_tokens for s in shards) != man["window_tokens"] or \
                sum(s.live_items for s in shards) != man["live_items"]:
            raise LedgerError("distributed manifest totals do not match its shards")
        return shards


# ------------------------------------------------------------------ lineage: collector <-> learner chain
CONTINUATION_FORMAT = 3
CONTINUATION_KIND = "rollout_ledger"
CONTINUATION_TP_LAYOUT = "tensor_parallel.communicator_rank_ascending.v1"
ROOT_LINEAGE = hashlib.sha256(b"ferrl.rollout-ledger.lineage-root.v1").hexdigest()


def _tensor_bytes(t: torch.Tensor) -> bytes:
    t = t.detach().contiguous().cpu()
    return t.reshape(-1).view(torch.uint8).numpy().tobytes() if t.numel() else b""


def state_digests(params: Sequence[torch.Tensor], optimizer, sampler_state: bytes, lora_recipe: Optional[str]) -> dict:
    """Digests of the learner's mutable state: ordered tensor schema, adapter values, Adam moments
    (independent of the step counter) and the opaque sampler state."""
    from .checkpoint import domain_sha256, tensor_schema_sha256
    ps = [p.detach() for p in params]
    return {
        "tensor_schema_sha256": tensor_schema_sha256(ps, lora_recipe),
        "adapter_sha256": domain_sha256("ferrl.rollout-ledger.adapter.v1", [_tensor_bytes(p) for p in ps]),
        "optimizer_sha256": domain_sha256("ferrl.rollout-ledger.optimizer.v1",
                                          [_tensor_bytes(t) for pair in zip(optimizer.m, optimizer.v) for t in pair]),
        "sampler_sha256": domain_sha256("ferrl.rollout-ledger.sampler.v1", [bytes(sampler_state)]),
    }


def lineage_sha256(parent_lineage: str, consumed_ledger_sha256: str, completed_step: int, post_state: dict) -> str:
    """The chain link a learner produces by consuming one window: binds the parent link, the exact
    ledger bytes consumed, the step completed and the state that resulted."""
    from .checkpoint import domain_sha256
    return domain_sha256("ferrl.rollout-ledger.lineage.v1",
                         [parent_lineage.encode(), consumed_ledger_sha256.encode(), str(int(completed_step)).encode()] +
                         [post_state[k].encode() for k in ("tensor_schema_sha256", "adapter_sha256", "optimizer_sha256",
                                                           "sampler_sha256")])


@dataclass
class LedgerContinuation:
    """What a learner hands to the next collector (and stores in its continuation checkpoint)."""
    completed_step: int
    policy_sha256: str
    trainer_config_sha256: str
    tensor_schema_sha256: str
    adapter_sha256: str
    optimizer_sha256: str
    sampler_sha256: str
    parent_lineage_sha256: str
    consumed_ledger_sha256: str
    lineage_sha256: str
    world_size: int = 1
    tensor_parallel_world_size: int = 1
    tensor_parallel_layout: str = CONTINUATION_TP_LAYOUT
    format_version: int = CONTINUATION_FORMAT
    kind: str = CONTINUATION_KIND

    def to_json(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_json(d: dict) -> "LedgerContinuation":
        try:
            c = LedgerContinuation(**d)
        except TypeError as e:
            raise LedgerError(f"malformed rollout-ledger continuation: {e}") from e
        if c.kind != CONTINUATION_KIND:
            raise LedgerError(f"continuation kind {c.kind!r} is not {CONTINUATION_KIND!r}")
        if not 1 <= c.format_version <= CONTINUATION_FORMAT:
            raise LedgerError(f"unsupported continuation format {c.format_version}")
        return c

    def verify(self) -> None:
        want = lineage_sha256(self.parent_lineage_sha256, self.consumed_ledger_sha256, self.completed_step, asdict(self))
        if want != self.lineage_sha256:
            raise LedgerError("continuation lineage does not follow from its parent, consumed ledger and state")

    def next_identity(self, optimizer_step: int) -> LedgerIdentity:
        """Identity of the window the next collector must write on top of this state."""
        return LedgerIdentity(self.trainer_config_sha256, self.policy_sha256, self.adapter_sha256, self.optimizer_sha256,
                              self.sampler_sha256, self.completed_step, optimizer_step, self.tensor_schema_sha256,
                              self.lineage_sha256)
