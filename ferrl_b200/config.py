"""Typed configuration: ``TrainerConfig`` and the single-file ``RunConfig``.

Reference: ``TrainerConfig`` fields/defaults/validation
(``crates/ferrl/src/trainer.rs:417-734``, ``:1092-1260``), ``ScalarSchedule``
(``:306-395``), and the CLI's strict JSON ``RunConfig`` with blocks ``policy``,
``data``, ``distributed``, ``tensor_parallel``, ``trimul``, ``run_health``,
``trainer`` (``crates/ferrl/src/bin/ferrl.rs:572-1258``): unknown fields are
rejected, ``trainer.eos_token_id`` is omitted / an integer / the string
``"none"`` (``null`` is rejected), and the validated config is re-serialised
canonically and SHA-256'd into a digest used for launch consensus and as a
checkpoint binding (``:1287-1319``).
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import math
import os
from dataclasses import dataclass, field
from typing import Any, Optional

from .grpo import ImportanceSamplingLevel, LossType, ScaleRewards


class ConfigError(ValueError):
    pass


def _require(cond: bool, msg: str) -> None:
    if not cond:
        raise ConfigError(msg)


@dataclass
class ScalarSchedule:
    """Piecewise-linear schedule over step indices; constant before the first
    and after the last point."""

    points: list  # list of (step:int, value:float)

    @staticmethod
    def constant(value: float) -> "ScalarSchedule":
        return ScalarSchedule([(0, float(value))])

    @staticmethod
    def linear(start: float, end: float, last_step: int) -> "ScalarSchedule":
        if last_step == 0:
            return ScalarSchedule.constant(end)
        return ScalarSchedule([(0, float(start)), (int(last_step), float(end))])

    def at(self, step: int) -> float:
        pts = self.points
        if step <= pts[0][0]:
            return pts[0][1]
        for (s0, v0), (s1, v1) in zip(pts, pts[1:]):
            if step <= s1:
                return v0 + (v1 - v0) * ((step - s0) / (s1 - s0))
        return pts[-1][1]

    def validate_nonnegative(self, label: str, steps: int) -> None:
        _require(len(self.points) > 0, f"{label}.points must not be empty")
        _require(self.points[0][0] == 0, f"{label}.points[0].step must be 0")
        prev = None
        for i, (s, v) in enumerate(self.points):
            _require(s < steps, f"{label}.points[{i}].step must be < trainer.steps")
            _require(math.isfinite(v) and v >= 0, f"{label}.points[{i}].value must be finite and >= 0")
            if prev is not None:
                _require(s > prev, f"{label}.points must be strictly increasing by step")
            prev = s

    def has_positive_value(self) -> bool:
        return any(v > 0 for _, v in self.points)

    def to_json(self):
        return {"points": [{"step": s, "value": v} for s, v in self.points]}

    @staticmethod
    def from_json(d) -> "ScalarSchedule":
        _strict(d, {"points"}, "schedule")
        pts = []
        for p in d["points"]:
            _strict(p, {"step", "value"}, "schedule point")
            pts.append((int(p["step"]), float(p["value"])))
        return ScalarSchedule(pts)


class RewardGroupScope:
    LOCAL = "local"
    DISTRIBUTED_SAME_PROMPT = "distributed_same_prompt"


@dataclass
class TrainerConfig:
    steps: int = 100
    group_size: int = 8
    max_new_tokens: int = 16
    temperature: float = 1.0
    mu: int = 1
    beta: float = 0.0
    beta_schedule: Optional[ScalarSchedule] = None
    clip_eps: float = 0.2
    clip_eps_high: Optional[float] = None
    importance_sampling_level: str = ImportanceSamplingLevel.TOKEN.value
    lr: float = 1e-3
    lr_schedule: Optional[ScalarSchedule] = None
    weight_decay: float = 0.0
    adam_beta1: float = 0.9
    adam_beta2: float = 0.999
    warmup_steps: int = 0
    max_grad_norm: Optional[float] = 1.0
    truncation_masking: bool = True
    tis: bool = False
    tis_imp_ratio_cap: float = 2.0
    loss_type: str = LossType.DAPO.value
    scale_rewards: str = ScaleRewards.GROUP.value
    reward_group_scope: str = RewardGroupScope.LOCAL
    grad_accum_steps: int = 1
    backward_microbatch_size: int = 0
    checkpoint_every: Optional[int] = None
    candidate_log_top_k: int = 0
    gpu_memory_probe: bool = False
    eos_token_id: Optional[int] = None
    # B200 additions (not in the reference): training-time nucleus and the
    # number of prompts decoded together per accumulation item.
    top_p: Optional[float] = None
    prompts_per_item: int = 1

    def validate(self) -> None:
        _require(self.steps >= 1, "steps must be >= 1 (0 performs no update)")
        _require(self.mu >= 1, "mu must be >= 1 (mu = 0 runs no inner update)")
        if self.reward_group_scope == RewardGroupScope.LOCAL:
            _require(self.group_size >= 2, "group_size must be >= 2 for local reward normalization")
        elif self.reward_group_scope == RewardGroupScope.DISTRIBUTED_SAME_PROMPT:
            _require(self.group_size >= 1, "group_size must be >= 1 for each distributed reward-group shard")
        else:
            raise ConfigError(f"unknown reward_group_scope {self.reward_group_scope!r}")
        _require(self.max_new_tokens >= 1, "max_new_tokens must be >= 1")
        _require(self.grad_accum_steps >= 1, "grad_accum_steps must be >= 1 (0 would never step the optimizer)")
        _require(self.prompts_per_item >= 1, "prompts_per_item must be >= 1")
        _require(math.isfinite(self.temperature) and self.temperature > 0, "temperature must be finite and > 0")
        _require(math.isfinite(self.lr) and self.lr >= 0, "lr must be finite and >= 0")
        _require(math.isfinite(self.weight_decay) and self.weight_decay >= 0, "weight_decay must be finite and >= 0")
        for n in ("adam_beta1", "adam_beta2"):
            v = getattr(self, n)
            _require(math.isfinite(v) and 0.0 <= v < 1.0, f"{n} must be finite and in [0, 1)")
        _require(math.isfinite(self.beta) and self.beta >= 0, "beta must be finite and >= 0")
        if self.beta_schedule is not None:
            self.beta_schedule.validate_nonnegative("beta_schedule", self.steps)
        _require(math.isfinite(self.clip_eps) and 0 <= self.clip_eps < 1.0,
                 "clip_eps must be finite and in [0, 1) (>= 1 disables the lower clip)")
        if self.lr_schedule is not None:
            self.lr_schedule.validate_nonnegative("lr_schedule", self.steps)
            _require(self.warmup_steps == 0,
                     "lr_schedule cannot be combined with warmup_steps; encode warmup as schedule points")
        if self.clip_eps_high is not None:
            _require(math.isfinite(self.clip_eps_high) and self.clip_eps_high >= 0,
                     "clip_eps_high must be finite and >= 0 when set")
        if self.max_grad_norm is not None:
            _require(math.isfinite(self.max_grad_norm) and self.max_grad_norm > 0,
                     "max_grad_norm must be finite and > 0 when set (use null to disable clipping)")
        if self.checkpoint_every is not None:
            _require(self.checkpoint_every >= 1, "checkpoint_every must be >= 1 when set (0 would checkpoint every step)")
        _require(math.isfinite(self.tis_imp_ratio_cap) and self.tis_imp_ratio_cap >= 1.0
                 and _finite_as_f32(self.tis_imp_ratio_cap),
                 "tis_imp_ratio_cap must be finite, >= 1, and remain finite when narrowed to the f32 TIS weight dtype "
                 "(a cap below 1 would down-weight exactly on-policy tokens)")
        _require(not (self.tis and self.importance_sampling_level == ImportanceSamplingLevel.SEQUENCE.value),
                 "tis is a token-level correction and cannot combine with sequence-level importance sampling (GSPO) "
                 "— pick one")
        if self.top_p is not None:
            _require(math.isfinite(self.top_p) and 0 < self.top_p <= 1.0, "top_p must be in (0, 1]")
        try:
            LossType(self.loss_type), ScaleRewards(self.scale_rewards)
            ImportanceSamplingLevel(self.importance_sampling_level)
        except ValueError as e:
            raise ConfigError(str(e)) from e

    def validate_reward_group_world(self, world_size: int) -> None:
        _require(world_size >= 1, "communicator world_size must be >= 1")
        eff = self.group_size if self.reward_group_scope == RewardGroupScope.LOCAL else self.group_size * world_size
        _require(eff >= 2, "effective reward-group size must be >= 2")

    def clip_eps_high_eff(self) -> float:
        return self.clip_eps if self.clip_eps_high is None else self.clip_eps_high

    def beta_at(self, step: int) -> float:
        return self.beta if self.beta_schedule is None else self.beta_schedule.at(step)

    def requires_reference_policy(self) -> bool:
        return self.beta > 0 if self.beta_schedule is None else self.beta_schedule.has_positive_value()

    def lr_at(self, step: int) -> float:
        if self.lr_schedule is not None:
            return self.lr_schedule.at(step)
        if self.warmup_steps == 0 or step + 1 >= self.warmup_steps:
            return self.lr
        return self.lr * ((step + 1) / self.warmup_steps)

    # -- JSON ---------------------------------------------------------
    def to_json(self) -> dict:
        d = dataclasses.asdict(self)
        for k in ("beta_schedule", "lr_schedule"):
            s = getattr(self, k)
            d[k] = None if s is None else s.to_json()
        return d

    @staticmethod
    def from_json(d: dict) -> "TrainerConfig":
        names = {f.name for f in dataclasses.fields(TrainerConfig)}
        _strict(d, names, "trainer")
        kw = dict(d)
        for k in ("beta_schedule", "lr_schedule"):
            if kw.get(k) is not None:
                kw[k] = ScalarSchedule.from_json(kw[k])
        cfg = TrainerConfig(**kw)
        cfg.validate()
        return cfg

    def digest(self) -> str:
        return canonical_digest(self.to_json(), b"ferrl-b200/trainer-config/v1")


def _finite_as_f32(x: float) -> bool:
    """Whether ``x`` rounds to a finite float32 (round-to-nearest, as a narrowing cast does)."""
    import struct
    try:
        return math.isfinite(struct.unpack("<f", struct.pack("<f", x))[0])
    except OverflowError:
        return False


def _strict(d: Any, allowed: set, what: str) -> None:
    if not isinstance(d, dict):
        raise ConfigError(f"{what} must be a JSON object")
    unknown = set(d.keys()) - set(allowed)
    if unknown:
        raise ConfigError(f"unknown field(s) in {what}: {sorted(unknown)}")


def canonical_json(obj: Any) -> bytes:
    return json.dumps(obj, sort_keys=True, separators=(",", ":"), ensure_ascii=True, allow_nan=False).encode()


def canonical_digest(obj: Any, domain: bytes) -> str:
    """Domain-separated SHA-256 of the canonical JSON form."""
    h = hashlib.sha256()
    h.update(domain + b"\0")
    h.update(canonical_json(obj))
    return h.hexdigest()


# ---------------------------------------------------------------- RunConfig
@dataclass
class PolicyCfg:
    lora_rank: int = 16
    lora_alpha: float = 32.0
    base_dtype: str = "f32"          # f32 | bf16 | f16
    base_quantization: str = "none"  # none | q8_0
    seed: int = 1234
    activation_checkpointing: bool = False
    memory_efficient_cached_gqa: bool = False
    lora_targets: str = "industrial"


@dataclass
class DataCfg:
    path: Optional[str] = None
    train_n: int = 64
    eval_n: int = 0
    seed: int = 7


@dataclass
class DistributedCfg:
    enabled: bool = False


@dataclass
class TensorParallelCfg:
    enabled: bool = False
    rank: int = 0
    world_size: int = 1
    # addition: keep the residual stream sharded over the token rows between the projections (reduce-scatter after
    # the row-parallel ones, all-gather in front of the column-parallel ones); model families that support it
    sequence_parallel: bool = False


@dataclass
class ExpertParallelCfg:
    """Experts of a sparse-MoE policy sharded over the data-parallel ranks (rank r owns experts
    ``[r*E/world, (r+1)*E/world)``); tokens travel to their experts and back through the
    dispatch/combine kernels.  Requires ``distributed.enabled`` (every rank still rolls out its
    own prompts) and an adapter recipe that leaves the routed experts frozen."""
    enabled: bool = False
    capacity_factor: float = 2.0


@dataclass
class RunConfig:
    task: str = "countdown"
    model_dir: str = ""
    device: str = "cpu"
    out_dir: str = "runs"
    launch_authentication: str = "signed"
    policy: PolicyCfg = field(default_factory=PolicyCfg)
    data: DataCfg = field(default_factory=DataCfg)
    distributed: DistributedCfg = field(default_factory=DistributedCfg)
    tensor_parallel: TensorParallelCfg = field(default_factory=TensorParallelCfg)
    expert_parallel: ExpertParallelCfg = field(default_factory=ExpertParallelCfg)
    trimul: dict = field(default_factory=dict)
    run_health: dict = field(default_factory=dict)
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    eos_selection: str = "checkpoint"  # checkpoint | explicit | disabled

    TASKS = ("countdown", "math", "trimul")

    @staticmethod
    def from_json(d: dict) -> "RunConfig":
        _strict(d, {"task", "model_dir", "device", "out_dir", "launch_authentication", "policy", "data",
                    "distributed", "tensor_parallel", "expert_parallel", "trimul", "run_health", "trainer"}, "run config")
        for req in ("task", "model_dir", "trainer"):
            _require(req in d, f"run config is missing required field {req!r}")
        t = dict(d["trainer"]) if isinstance(d["trainer"], dict) else d["trainer"]
        _require(isinstance(t, dict), "trainer must be a JSON object")
        eos_sel = "checkpoint"
        if "eos_token_id" in t:
            raw = t["eos_token_id"]
            if isinstance(raw, bool) or raw is None:
                raise ConfigError("trainer.eos_token_id must be omitted for checkpoint auto-resolution, an "
                                  "integer override, or the string \"none\"; null is not an explicit mode")
            if isinstance(raw, int) and 0 <= raw < 2 ** 32:
                eos_sel = "explicit"
            elif raw == "none":
                eos_sel = "disabled"
                t["eos_token_id"] = None
            else:
                raise ConfigError("trainer.eos_token_id must be an integer override or the string \"none\"")

        def block(cls, key):
            raw = d.get(key, {})
            _strict(raw, {f.name for f in dataclasses.fields(cls)}, key)
            return cls(**raw)

        cfg = RunConfig(task=d["task"], model_dir=d["model_dir"], device=d.get("device", "cpu"),
                        out_dir=d.get("out_dir", "runs"),
                        launch_authentication=d.get("launch_authentication", "signed"),
                        policy=block(PolicyCfg, "policy"), data=block(DataCfg, "data"),
                        distributed=block(DistributedCfg, "distributed"),
                        tensor_parallel=block(TensorParallelCfg, "tensor_parallel"),
                        expert_parallel=block(ExpertParallelCfg, "expert_parallel"),
                        trimul=dict(d.get("trimul", {})), run_health=dict(d.get("run_health", {})),
                        trainer=TrainerConfig.from_json(t), eos_selection=eos_sel)
        cfg.validate()
        return cfg

    @staticmethod
    def load(path: str) -> "RunConfig":
        try:
            with open(path, encoding="utf-8") as f:
                raw = json.load(f)
        except OSError as e:
            raise ConfigError(f"cannot read run config {path}: {e}") from e
        except json.JSONDecodeError as e:
            raise ConfigError(f"run config {path} is not valid JSON: {e}") from e
        return RunConfig.from_json(raw)

    def validate(self) -> None:
        _require(self.task in self.TASKS, f"task must be one of {self.TASKS}, got {self.task!r}")
        _require(isinstance(self.model_dir, str) and self.model_dir != "", "model_dir must be set")
        _require(self.policy.base_dtype in ("f32", "bf16", "f16"), "policy.base_dtype must be f32, bf16 or f16")
        _require(self.policy.base_quantization in ("none", "q8_0"), "policy.base_quantization must be none or q8_0")
        _require(self.policy.lora_rank >= 1, "policy.lora_rank must be >= 1")
        _require(self.launch_authentication in ("signed", "unsigned_development"),
                 "launch_authentication must be signed or unsigned_development")
        tp = self.tensor_parallel
        if tp.enabled:
            _require(tp.world_size >= 2 and 0 <= tp.rank < tp.world_size,
                     "tensor_parallel needs world_size >= 2 and 0 <= rank < world_size")
            _require(not self.distributed.enabled,
                     "data-parallel and tensor-parallel launches cannot be combined")
        if self.expert_parallel.enabled:
            _require(self.distributed.enabled and not tp.enabled,
                     "expert_parallel shards experts over data-parallel ranks: it needs distributed.enabled and no tensor_parallel")
            _require(self.expert_parallel.capacity_factor >= 1.0, "expert_parallel.capacity_factor must be >= 1")
        self.trainer.validate()
        # the remaining rules follow the reference's launch validation (crates/ferrl/src/bin/ferrl.rs:1260-1380)
        if (not self.distributed.enabled and self.trainer.reward_group_scope == RewardGroupScope.DISTRIBUTED_SAME_PROMPT
                and self.trainer.group_size < 2):
            raise ConfigError("distributed_same_prompt group_size = 1 requires a live data-parallel world of at least two ranks")
        try:
            import torch
            from .models.lora import validated_lora_scale
            validated_lora_scale(self.policy.lora_rank, self.policy.lora_alpha,
                                 {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}[self.policy.base_dtype])
        except ValueError as e:
            raise ConfigError(f"invalid policy LoRA scale: {e}") from e
        if self.task in ("countdown", "trimul"):
            _require(self.data.train_n >= 1, f"task {self.task!r} requires data.train_n >= 1")
        if self.task == "trimul":
            self._validate_trimul()
        from .run_health import validate_run_health
        validate_run_health(self.run_health, self.trainer)

    TRIMUL_CASE_SEED_MAX = (1 << 32) - 1

    def _validate_trimul(self) -> None:
        t = self.trimul
        seed = t.get("secret_seed", 0)
        _require(isinstance(seed, int) and not isinstance(seed, bool) and 0 <= seed <= self.TRIMUL_CASE_SEED_MAX,
                 f"trimul.secret_seed must be between 0 and {self.TRIMUL_CASE_SEED_MAX}")
        held = t.get("held_out_secret_seed")
        if self.data.eval_n == 0:
            _require(held is None, "trimul.held_out_secret_seed requires data.eval_n >= 1")
        else:
            _require(held is not None, "TriMul held-out eval requires trimul.held_out_secret_seed")
            _require(isinstance(held, int) and not isinstance(held, bool) and 0 <= held <= self.TRIMUL_CASE_SEED_MAX
                     and held != seed,
                     "trimul.held_out_secret_seed must be in the u32 range and differ from trimul.secret_seed")
        tier = t.get("verifier_isolation_tier", "same_uid_apptainer_v1")
        if tier == "same_uid_apptainer_v1":
            _require(t.get("verifier_executor_socket") is None,
                     "trimul.verifier_executor_socket is valid only with \"dedicated_uid_service_v1\"; same-UID "
                     "verification never falls back to or contacts the executor service")
            bin_ = t.get("verifier_apptainer_bin")
            _require(bin_ is None or os.path.isabs(str(bin_)), "trimul.verifier_apptainer_bin must be an absolute path")
        elif tier == "dedicated_uid_service_v1":
            _require(t.get("verifier_apptainer_bin") is None,
                     "trimul.verifier_apptainer_bin is valid only with \"same_uid_apptainer_v1\"; the dedicated "
                     "service owns its Apptainer executable")
        else:
            raise ConfigError(f"unknown trimul.verifier_isolation_tier {tier!r}")

    def to_json(self, *, for_consensus: bool = False) -> dict:
        t = self.trainer.to_json()
        if self.eos_selection == "checkpoint":
            t.pop("eos_token_id", None)
        elif self.eos_selection == "disabled":
            t["eos_token_id"] = "none"
        tp = dataclasses.asdict(self.tensor_parallel)
        if for_consensus:
            tp.pop("rank")  # the only field allowed to differ between ranks
        return {"task": self.task, "model_dir": self.model_dir, "device": self.device, "out_dir": self.out_dir,
                "launch_authentication": self.launch_authentication, "policy": dataclasses.asdict(self.policy),
                "data": dataclasses.asdict(self.data), "distributed": dataclasses.asdict(self.distributed),
                "tensor_parallel": tp, "trimul": self.trimul, "run_health": self.run_health, "trainer": t,
                **({"expert_parallel": dataclasses.asdict(self.expert_parallel)} if self.expert_parallel.enabled else {})}

    def digest(self) -> str:
        return canonical_digest(self.to_json(for_consensus=True), b"ferrl-b200/run-config/v1")
