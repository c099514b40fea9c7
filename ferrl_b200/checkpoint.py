"""Checkpoint / resume: adapters, optimizer moments, sampler state, manifest.

On-disk layout (reference ``crates/ferrl/src/checkpoint.rs:192-196``)::

    <run>/checkpoints/step-N/adapter.safetensors     keys lora.00000 ...
                             optimizer.safetensors   keys m.00000 / v.00000 ...
                             manifest.json           written last

Format version 4 (``:208``). The manifest (``:370-412``) records step, var
count, optimizer step counter, sampler state bytes, LoRA recipe and an
``ordinary_checkpoint`` identity: payload SHA-256s, tensor-schema digest and
the binding digests (frozen policy, trainer config).  Digests are
length-prefixed and domain-separated (``:447-456``).  Publication is staged:
payloads are written and fsynced into a temp directory, ``manifest.json`` goes
last, the directory is renamed into place atomically under an advisory writer
lock (``:649-1275``); an existing ``step-N`` is never replaced.  Loading
verifies every digest and the binding *before* mutating any live state
(``:2236-2348``).  ``latest_checkpoint`` picks the highest complete step and
treats a newer malformed one as an error rather than silently falling back
(``:2436``).
"""
from __future__ import annotations

import fcntl
import hashlib
import json
import os
import re
import shutil
import struct
from dataclasses import dataclass, field
from typing import Optional, Sequence

import torch

from .optim import OptimizerState

ADAPTER_FILE = "adapter.safetensors"
OPTIMIZER_FILE = "optimizer.safetensors"
MANIFEST_FILE = "manifest.json"
LOCK_SUFFIX = ".writer-lock"                   # reference checkpoint.rs WRITER_LOCK_SUFFIX
TOPOLOGY_FILE = "topology.json"                # readable copy of what trainer_config_sha256 also binds
ORDINARY_KIND = "ordinary"
_DOMAIN = "ferrl.ordinary-checkpoint."         # digest domains of the reference (checkpoint.rs:447-540)
FORMAT_VERSION = 4
MIN_READ_VERSION = 4
_STEP_RE = re.compile(r"^step-(\d+)$")


class CheckpointError(RuntimeError):
    pass


class CheckpointMismatch(CheckpointError):
    pass


def domain_sha256(domain: str, fields: Sequence[bytes]) -> str:
    h = hashlib.sha256()
    h.update(struct.pack("<Q", len(domain)))
    h.update(domain.encode())
    for f in fields:
        h.update(struct.pack("<Q", len(f)))
        h.update(f)
    return h.hexdigest()


def _validate_sha(label: str, s: str) -> None:
    if not (isinstance(s, str) and len(s) == 64 and all(c in "0123456789abcdef" for c in s)):
        raise CheckpointMismatch(f"{label} must be 64 lowercase hexadecimal characters")


@dataclass(frozen=True)
class CheckpointBinding:
    frozen_policy_sha256: str
    trainer_config_sha256: str
    lora_recipe: Optional[str] = None

    def __post_init__(self):
        _validate_sha("frozen_policy_sha256", self.frozen_policy_sha256)
        _validate_sha("trainer_config_sha256", self.trainer_config_sha256)


def var_key(i: int) -> str:
    return f"lora.{i:05d}"


def moment_key(kind: str, i: int) -> str:
    return f"{kind}.{i:05d}"


_CANDLE_DTYPE = {torch.float32: "f32", torch.float64: "f64", torch.bfloat16: "bf16", torch.float16: "f16",
                 torch.uint8: "u8", torch.int64: "i64", torch.int32: "i32", torch.int16: "i16"}


def _compact_json(obj) -> bytes:
    """The byte form ``serde_json::to_vec`` produces: no whitespace, keys in insertion order,
    UTF-8 written raw."""
    return json.dumps(obj, separators=(",", ":"), ensure_ascii=False).encode("utf-8")


def _dtype_name(dt: torch.dtype) -> str:
    try:
        return _CANDLE_DTYPE[dt]
    except KeyError:
        raise CheckpointMismatch(f"dtype {dt} has no checkpoint schema name") from None


def tensor_schema_sha256(tensors: Sequence[torch.Tensor], lora_recipe: Optional[str]) -> str:
    """Digest of ``(recipe, [(key, dims, dtype), ...])`` as compact JSON (reference
    checkpoint.rs ``tensor_schema_sha256``): shape-aliased recipes get different identities."""
    schema = [[var_key(i), [int(d) for d in t.shape], _dtype_name(t.dtype)] for i, t in enumerate(tensors)]
    return domain_sha256(_DOMAIN + "tensor-schema.v1", [_compact_json([lora_recipe, schema])])


def adapter_payload_sha256(data: bytes) -> str:
    return domain_sha256(_DOMAIN + "adapter.v1", [data])


def optimizer_payload_sha256(step_t: int, data: bytes) -> str:
    """The Adam bias-correction counter is bound into the optimizer digest, so an edited
    ``optimizer_step_t`` cannot pass verification."""
    if not 0 <= int(step_t) < 1 << 64:
        raise CheckpointMismatch("optimizer step_t does not fit the checkpoint's u64 identity")
    return domain_sha256(_DOMAIN + "optimizer.v1", [struct.pack("<Q", int(step_t)), data])


def sampler_payload_sha256(data: bytes) -> str:
    return domain_sha256(_DOMAIN + "sampler.v1", [data])


def state_envelope_sha256(format_version: int, kind: str, step: int, num_vars: int, lora_recipe: Optional[str],
                          optimizer_step_t: int, optimizer_num_vars: int, ident: dict) -> str:
    """Root digest over version/kind, step, counts, recipe, the two immutable identities and every
    mutable payload digest, in the reference's field order (checkpoint.rs ``OrdinaryCheckpointEnvelope``)."""
    env = {"format_version": int(format_version), "kind": kind, "step": int(step), "num_vars": int(num_vars),
           "lora_recipe": lora_recipe, "optimizer_step_t": int(optimizer_step_t),
           "optimizer_num_vars": int(optimizer_num_vars)}
    for k in ("frozen_policy_sha256", "trainer_config_sha256", "tensor_schema_sha256", "adapter_sha256",
              "optimizer_sha256", "sampler_sha256"):
        env[k] = ident[k]
    return domain_sha256(_DOMAIN + "state-envelope.v1", [_compact_json(env)])


def bound_trainer_config_sha256(trainer_config_sha256: str, world_size: int, topology: str) -> str:
    """The manifest's ``trainer_config_sha256`` covers the learner-semantic config AND the topology
    (the reference's manifest has no world/topology fields and rejects unknown ones): this is the
    caller's config digest extended by world size and topology name."""
    return domain_sha256(_DOMAIN + "trainer-config-topology.v1",
                         [trainer_config_sha256.encode(), topology.encode(), struct.pack("<Q", int(world_size))])


def _read_bytes(path: str) -> bytes:
    with open(path, "rb") as f:
        return f.read()


def _file_sha256(path: str) -> str:
    h = hashlib.sha256()
    with open(path, "rb") as f:
        while True:
            b = f.read(1 << 20)
            if not b:
                break
            h.update(b)
    return h.hexdigest()


def _fsync_file(path: str) -> None:
    fd = os.open(path, os.O_RDONLY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def _fsync_dir(path: str) -> None:
    fd = os.open(path, os.O_RDONLY | os.O_DIRECTORY)
    try:
        os.fsync(fd)
    finally:
        os.close(fd)


def _save_tensors(path: str, named: dict) -> None:
    from safetensors.torch import save_file
    save_file({k: v.detach().to("cpu").contiguous() for k, v in named.items()}, path)
    _fsync_file(path)


def _load_tensors(path: str) -> dict:
    from safetensors.torch import load_file
    try:
        return load_file(path)
    except Exception as e:  # noqa: BLE001 - any parse failure is a corrupt payload
        raise CheckpointMismatch(f"cannot parse {path}: {e}") from e


@dataclass
class CheckpointManifest:
    """Field set of the reference's ``CheckpointManifest`` (checkpoint.rs:370-412), which rejects
    unknown fields; world size and topology are therefore not manifest fields (see
    ``bound_trainer_config_sha256`` and the ``topology.json`` side file)."""
    format_version: int
    step: int
    num_vars: int
    optimizer_step_t: Optional[int] = None
    optimizer_num_vars: Optional[int] = None
    sampler_state: Optional[list] = None      # bytes as a list of ints (JSON friendly)
    lora_recipe: Optional[str] = None
    rollout_ledger_continuation: Optional[dict] = None
    ordinary_checkpoint: Optional[dict] = None
    world_size: int = 1                       # from topology.json, not serialised into manifest.json
    topology: str = "dp"

    FIELDS = ("format_version", "step", "num_vars", "optimizer_step_t", "optimizer_num_vars", "sampler_state",
              "lora_recipe", "rollout_ledger_continuation", "ordinary_checkpoint")
    IDENTITY_FIELDS = ("kind", "frozen_policy_sha256", "trainer_config_sha256", "tensor_schema_sha256",
                       "adapter_sha256", "optimizer_sha256", "sampler_sha256", "state_envelope_sha256")

    def to_json(self) -> dict:
        return {k: getattr(self, k) for k in self.FIELDS}

    @staticmethod
    def from_json(d: dict) -> "CheckpointManifest":
        if not isinstance(d, dict):
            raise CheckpointMismatch("manifest is not a JSON object")
        unknown = set(d) - set(CheckpointManifest.FIELDS)
        if unknown:
            raise CheckpointMismatch(f"manifest has unknown fields {sorted(unknown)}")
        for req in ("format_version", "step", "num_vars"):
            if req not in d:
                raise CheckpointMismatch(f"manifest is missing {req}")
        for k in ("format_version", "step", "num_vars"):
            if not isinstance(d[k], int) or isinstance(d[k], bool) or d[k] < 0:
                raise CheckpointMismatch(f"manifest field {k} must be a non-negative integer")
        ident = d.get("ordinary_checkpoint")
        if ident is not None:
            if not isinstance(ident, dict) or set(ident) != set(CheckpointManifest.IDENTITY_FIELDS):
                raise CheckpointMismatch("ordinary_checkpoint identity has missing or unknown fields")
            for k in CheckpointManifest.IDENTITY_FIELDS[1:]:
                _validate_sha(k, ident[k])
        return CheckpointManifest(**d)

    def sampler_bytes(self) -> Optional[bytes]:
        return None if self.sampler_state is None else bytes(self.sampler_state)


@dataclass
class LoadedCheckpoint:
    manifest: CheckpointManifest
    adapters: list
    optimizer: Optional[OptimizerState]
    path: str


def step_dir(checkpoints_dir: str, step: int) -> str:
    return os.path.join(checkpoints_dir, f"step-{step}")


class _WriterLock:
    def __init__(self, path: str):
        self.path = path
        self.fd = None

    def __enter__(self):
        self.fd = os.open(self.path, os.O_WRONLY | os.O_CREAT, 0o644)
        try:
            fcntl.flock(self.fd, fcntl.LOCK_EX | fcntl.LOCK_NB)
        except OSError as e:
            os.close(self.fd)
            raise CheckpointError(f"another writer holds {self.path}") from e
        return self

    def __exit__(self, *exc):
        fcntl.flock(self.fd, fcntl.LOCK_UN)
        os.close(self.fd)
        return False


def save_checkpoint(checkpoints_dir: str, step: int, adapters: Sequence[torch.Tensor],
                    optimizer: Optional[OptimizerState], sampler_state: Optional[bytes],
                    binding: CheckpointBinding, *, world_size: int = 1, topology: str = "dp",
                    fault_hook=None, continuation: Optional[dict] = None) -> str:
    """Stage, fsync, publish atomically.  ``fault_hook(stage_name)`` lets tests
    inject host-side failures between stages.  ``continuation`` (the JSON form of a
    ``ledger.LedgerContinuation``) marks the checkpoint as the post-state of a separated
    collector/learner chain: it is bound into the manifest and, like every checkpoint here,
    never replaces an existing ``step-N`` (reference checkpoint.rs:1631)."""
    os.makedirs(checkpoints_dir, exist_ok=True)
    final = step_dir(checkpoints_dir, step)
    if os.path.exists(final):
        raise CheckpointError(f"{final} already exists; a published checkpoint is never replaced")
    with _WriterLock(final + LOCK_SUFFIX):
        stage = final + f".staging-{os.getpid()}"
        if os.path.exists(stage):
            shutil.rmtree(stage)
        os.makedirs(stage)
        try:
            ap = os.path.join(stage, ADAPTER_FILE)
            _save_tensors(ap, {var_key(i): t for i, t in enumerate(adapters)})
            if fault_hook:
                fault_hook("adapter_written")
            op = os.path.join(stage, OPTIMIZER_FILE)
            named = {}
            if optimizer is not None:
                for i, (m, v) in enumerate(zip(optimizer.m, optimizer.v)):
                    named[moment_key("m", i)] = m
                    named[moment_key("v", i)] = v
            _save_tensors(op, named)
            if fault_hook:
                fault_hook("optimizer_written")
            sampler = sampler_state or b""
            step_t = optimizer.step if optimizer else 0
            n_opt = len(optimizer.m) if optimizer else 0
            ident = {
                "kind": ORDINARY_KIND,
                "frozen_policy_sha256": binding.frozen_policy_sha256,
                "trainer_config_sha256": bound_trainer_config_sha256(binding.trainer_config_sha256, world_size, topology),
                "tensor_schema_sha256": tensor_schema_sha256(adapters, binding.lora_recipe),
                "adapter_sha256": adapter_payload_sha256(_read_bytes(ap)),
                "optimizer_sha256": optimizer_payload_sha256(step_t, _read_bytes(op)),
                "sampler_sha256": sampler_payload_sha256(sampler),
            }
            ident["state_envelope_sha256"] = state_envelope_sha256(
                FORMAT_VERSION, ORDINARY_KIND, step, len(adapters), binding.lora_recipe, step_t, n_opt, ident)
            man = CheckpointManifest(FORMAT_VERSION, step, len(adapters), step_t, n_opt,
                                     list(sampler) if sampler_state is not None else None,
                                     binding.lora_recipe,
                                     dict(continuation) if continuation is not None else None, ident)
            tp = os.path.join(stage, TOPOLOGY_FILE)
            with open(tp, "w", encoding="utf-8") as f:
                json.dump({"world_size": int(world_size), "topology": topology}, f, sort_keys=True)
                f.flush()
                os.fsync(f.fileno())
            mp = os.path.join(stage, MANIFEST_FILE)
            with open(mp, "w", encoding="utf-8") as f:
                json.dump(man.to_json(), f, sort_keys=True)
                f.flush()
                os.fsync(f.fileno())
            if fault_hook:
                fault_hook("manifest_written")
            _fsync_dir(stage)
            os.rename(stage, final)
            _fsync_dir(checkpoints_dir)
        except BaseException:
            shutil.rmtree(stage, ignore_errors=True)
            raise
    try:
        os.unlink(final + LOCK_SUFFIX)
    except OSError:
        pass
    return final


def read_manifest(path: str) -> CheckpointManifest:
    mp = os.path.join(path, MANIFEST_FILE)
    try:
        with open(mp, encoding="utf-8") as f:
            man = CheckpointManifest.from_json(json.load(f))
    except FileNotFoundError:
        raise CheckpointMismatch(f"{path} has no manifest (incomplete checkpoint)") from None
    except json.JSONDecodeError as e:
        raise CheckpointMismatch(f"{mp} is not valid JSON: {e}") from e
    except TypeError as e:
        raise CheckpointMismatch(f"{mp} is malformed: {e}") from e
    tp = os.path.join(path, TOPOLOGY_FILE)
    if os.path.exists(tp):
        try:
            with open(tp, encoding="utf-8") as f:
                t = json.load(f)
            man.world_size, man.topology = int(t["world_size"]), str(t["topology"])
        except (ValueError, KeyError, TypeError) as e:
            raise CheckpointMismatch(f"{tp} is malformed: {e}") from e
    return man


def prepare_checkpoint(path: str, binding: Optional[CheckpointBinding], expected_shapes: Optional[Sequence] = None,
                       *, world_size: Optional[int] = None, topology: Optional[str] = None) -> LoadedCheckpoint:
    """Read and verify everything; touches no live state.  Order: version and kind, the state
    envelope (so an edited step / counter / count field fails before any payload is read), payload
    digests, binding, topology, tensor keys + schema + shapes (adapters and both Adam moments)."""
    man = read_manifest(path)
    if not (MIN_READ_VERSION <= man.format_version <= FORMAT_VERSION):
        raise CheckpointMismatch(f"unsupported checkpoint format {man.format_version}")
    ident = man.ordinary_checkpoint
    if ident is None:
        raise CheckpointMismatch("manifest carries no checkpoint identity")
    if ident.get("kind") != ORDINARY_KIND:
        raise CheckpointMismatch(f"checkpoint kind {ident.get('kind')!r} is not {ORDINARY_KIND!r}")
    if man.optimizer_step_t is None or man.optimizer_num_vars is None:
        raise CheckpointMismatch("ordinary checkpoint is missing optimizer_step_t / optimizer_num_vars")
    if state_envelope_sha256(man.format_version, ident["kind"], man.step, man.num_vars, man.lora_recipe,
                             man.optimizer_step_t, man.optimizer_num_vars, ident) != ident["state_envelope_sha256"]:
        raise CheckpointMismatch("ordinary checkpoint state-envelope digest mismatch")
    ap, op = os.path.join(path, ADAPTER_FILE), os.path.join(path, OPTIMIZER_FILE)
    for p in (ap, op):
        if not os.path.exists(p):
            raise CheckpointMismatch(f"missing payload {p}")
    if adapter_payload_sha256(_read_bytes(ap)) != ident["adapter_sha256"]:
        raise CheckpointMismatch(f"{ADAPTER_FILE} does not match its recorded SHA-256")
    if optimizer_payload_sha256(man.optimizer_step_t, _read_bytes(op)) != ident["optimizer_sha256"]:
        raise CheckpointMismatch(f"{OPTIMIZER_FILE} (with its step counter) does not match its recorded SHA-256")
    sampler = man.sampler_bytes() or b""
    if sampler_payload_sha256(sampler) != ident["sampler_sha256"]:
        raise CheckpointMismatch("sampler state does not match its recorded digest")
    if world_size is not None and man.world_size != world_size:
        raise CheckpointMismatch(f"checkpoint world size {man.world_size} differs from the live world {world_size}")
    if topology is not None and man.topology != topology:
        raise CheckpointMismatch(f"checkpoint topology {man.topology!r} differs from {topology!r}")
    if binding is not None:
        if ident["frozen_policy_sha256"] != binding.frozen_policy_sha256:
            raise CheckpointMismatch("checkpoint was written for a different frozen policy")
        if ident["trainer_config_sha256"] != bound_trainer_config_sha256(binding.trainer_config_sha256,
                                                                        man.world_size, man.topology):
            raise CheckpointMismatch("checkpoint was written under a different trainer config or topology")
        if man.lora_recipe != binding.lora_recipe:
            raise CheckpointMismatch(f"checkpoint LoRA recipe {man.lora_recipe!r} differs from "
                                     f"the live recipe {binding.lora_recipe!r}")
    at = _load_tensors(ap)
    adapters = []
    for i in range(man.num_vars):
        k = var_key(i)
        if k not in at:
            raise CheckpointMismatch(f"adapter payload is missing {k}")
        adapters.append(at[k])
    if len(at) != man.num_vars:
        raise CheckpointMismatch("adapter payload has unexpected extra tensors")
    if tensor_schema_sha256(adapters, man.lora_recipe) != ident["tensor_schema_sha256"]:
        raise CheckpointMismatch("tensor schema digest mismatch")
    if expected_shapes is not None:
        if len(expected_shapes) != len(adapters):
            raise CheckpointMismatch(f"checkpoint has {len(adapters)} tensors, live model has {len(expected_shapes)}")
        for i, (t, s) in enumerate(zip(adapters, expected_shapes)):
            if tuple(t.shape) != tuple(s):
                raise CheckpointMismatch(f"tensor {i} shape {tuple(t.shape)} differs from live {tuple(s)}")
    opt = None
    ot = _load_tensors(op)
    n_opt = man.optimizer_num_vars
    if len(ot) != 2 * n_opt:
        raise CheckpointMismatch(f"optimizer payload holds {len(ot)} tensors, manifest promises {2 * n_opt}")
    if n_opt not in (0, man.num_vars):
        raise CheckpointMismatch(f"optimizer covers {n_opt} tensors, the adapter has {man.num_vars}")
    if n_opt:
        m, v = [], []
        for i in range(n_opt):
            for kind, dst in (("m", m), ("v", v)):
                k = moment_key(kind, i)
                if k not in ot:
                    raise CheckpointMismatch(f"optimizer payload is missing {k}")
                if tuple(ot[k].shape) != tuple(adapters[i].shape):
                    raise CheckpointMismatch(f"optimizer tensor {k} shape {tuple(ot[k].shape)} differs from "
                                             f"its adapter tensor {tuple(adapters[i].shape)}")
                dst.append(ot[k])
        opt = OptimizerState(int(man.optimizer_step_t), m, v)
    return LoadedCheckpoint(man, adapters, opt, path)


def load_checkpoint(path: str, binding: Optional[CheckpointBinding], params: Sequence[torch.nn.Parameter],
                    **kw) -> LoadedCheckpoint:
    """Verify, then copy adapter values into ``params`` (all-or-nothing)."""
    lc = prepare_checkpoint(path, binding, [tuple(p.shape) for p in params], **kw)
    with torch.no_grad():
        for p, t in zip(params, lc.adapters):
            p.copy_(t.to(p.dtype))
    return lc


def latest_rollout_ledger_continuation(checkpoints_dir: str) -> Optional[tuple[int, str, dict]]:
    """Highest ``step-N`` whose manifest carries a rollout-ledger continuation:
    ``(step, path, continuation)``.  Ordinary checkpoints are skipped, so the two kinds are
    discovered separately."""
    if not os.path.isdir(checkpoints_dir):
        return None
    best = None
    for name in os.listdir(checkpoints_dir):
        m = _STEP_RE.match(name)
        if not m:
            continue
        path = os.path.join(checkpoints_dir, name)
        if not os.path.exists(os.path.join(path, MANIFEST_FILE)):
            continue
        man = read_manifest(path)
        c = man.rollout_ledger_continuation
        if c is None:
            continue
        if c.get("kind") != "rollout_ledger":
            raise CheckpointMismatch(f"{path} carries a continuation of unknown kind {c.get('kind')!r}")
        if best is None or int(m.group(1)) > best[0]:
            best = (int(m.group(1)), path, c)
    return best


def latest_checkpoint(checkpoints_dir: str) -> Optional[tuple[int, str]]:
    """Highest complete ordinary ``step-N``; a newer malformed final directory is an error.
    Directories whose manifest carries a rollout-ledger continuation belong to the separated
    collector/learner chain and are discovered by ``latest_rollout_ledger_continuation`` only."""
    if not os.path.isdir(checkpoints_dir):
        return None
    steps = []
    for name in os.listdir(checkpoints_dir):
        m = _STEP_RE.match(name)
        if m and os.path.isdir(os.path.join(checkpoints_dir, name)):
            steps.append(int(m.group(1)))
    for best in sorted(steps, reverse=True):
        path = step_dir(checkpoints_dir, best)
        man = read_manifest(path)  # raises CheckpointMismatch if the newest is malformed
        if man.rollout_ledger_continuation is not None:
            continue
        if man.step != best:
            raise CheckpointMismatch(f"{path} manifest records step {man.step}")
        return best, path
    return None


def save_adapter(path: str, adapters: Sequence[torch.Tensor], lora_recipe: Optional[str] = None) -> None:
    """Bare adapter file for evaluation (no optimizer, no manifest)."""
    from safetensors.torch import save_file
    tmp = path + ".tmp"
    save_file({var_key(i): t.detach().cpu().contiguous() for i, t in enumerate(adapters)}, tmp,
              metadata={"lora_recipe": lora_recipe or "", "format": "ferrl-b200-adapter-v1"})
    _fsync_file(tmp)
    os.rename(tmp, path)


def load_adapter(path: str, params: Sequence[torch.nn.Parameter], lora_recipe: Optional[str] = None) -> None:
    from safetensors import safe_open
    try:
        with safe_open(path, framework="pt") as f:
            meta = f.metadata() or {}
            tensors = {k: f.get_tensor(k) for k in f.keys()}
    except Exception as e:  # noqa: BLE001
        raise CheckpointMismatch(f"cannot read adapter {path}: {e}") from e
    if lora_recipe is not None and meta.get("lora_recipe", "") not in ("", lora_recipe):
        raise CheckpointMismatch(f"adapter recipe {meta.get('lora_recipe')!r} differs from live {lora_recipe!r}")
    if len(tensors) != len(params):
        raise CheckpointMismatch(f"adapter has {len(tensors)} tensors, live model has {len(params)}")
    vals = []
    for i, p in enumerate(params):
        t = tensors.get(var_key(i))
        if t is None or tuple(t.shape) != tuple(p.shape):
            raise CheckpointMismatch(f"adapter tensor {i} is missing or has the wrong shape")
        vals.append(t)
    with torch.no_grad():
        for p, t in zip(params, vals):
            p.copy_(t.to(p.dtype))
