"""Discovery SDK: the small stable surface for "train a policy on a verifiable task, verify its
best candidates independently, and publish a winning artifact".

Reference ``crates/ferrl/src/discovery.rs``: task identity ``:184-232``, metric contract and
report ``:361-600``, final evidence / candidate verification ``:622-770``, ``DiscoveryTask``
``:782-831``, ``DiscoveryConfig`` + builder ``:835-1029``, ``Discovery::run`` ``:1064-1140``,
outcomes (verified / no win / preempted) ``:1172-1380``, candidate selection ``:1714-1821``,
manifest-last artifact publication ``:1857-2040``.  The engine underneath is
``ferrl_b200.orchestration``; this module fixes a narrow, typed entry point.

Flow: validate the configuration before anything is loaded (output must not exist, must not
contain the runs root) -> train with the fixed recipe -> held-out evaluation -> every
authenticated candidate (best search reward first) goes to the task's ``verify_candidate``;
a candidate wins when the verifier measured it, proved held-out correctness and its metric beats
the launch-frozen baseline by strictly more than the materiality margin; among winners the
strongest metric is kept (ties keep the better-ranked candidate) -> the bundle
``artifact.json``, ``launch.json``, ``eval-report.json``, ``candidate.json``,
``verifier-evidence.json`` is staged, and ``manifest.json`` (contract tag, identities, SHA-256
of every file) is written last before the directory is renamed into place.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
from dataclasses import asdict, dataclass, field
from typing import Any, Callable, Optional, Sequence

from .config import PolicyCfg, RunConfig, TrainerConfig
from .orchestration import TrainOutcome, run_cli_train_setup
from .rewards import RewardFn, Sample

ARTIFACT_CONTRACT = "ferrl.discovery-artifact.v1"
HELD_OUT_REPORT_CONTRACT = "ferrl.discovery-held-out-report.v1"
VERIFIER_EVIDENCE_CONTRACT = "ferrl.discovery-verifier-evidence.v1"
ARTIFACT_FILES = ("artifact.json", "launch.json", "eval-report.json", "candidate.json", "verifier-evidence.json")
ARTIFACT_MANIFEST_FILE = "manifest.json"
METRIC_LABEL_MAX_BYTES = 128
HIGHER_IS_BETTER, LOWER_IS_BETTER = "higher_is_better", "lower_is_better"


class DiscoveryError(RuntimeError):
    pass


class InvalidConfiguration(DiscoveryError, ValueError):
    pass


class InvalidFinalEvidence(DiscoveryError, ValueError):
    pass


class TaskVerificationError(DiscoveryError):
    """The final verifier could not produce an honest decision (infrastructure, sandbox or
    benchmark failure): the run aborts instead of counting the candidate as rejected."""


def _label(what: str, value: str) -> None:
    if not isinstance(value, str) or not value.strip() or value.strip() != value \
            or len(value.encode()) > METRIC_LABEL_MAX_BYTES or any(ord(c) < 32 or ord(c) == 127 for c in value):
        raise InvalidFinalEvidence(f"{what} must be 1..={METRIC_LABEL_MAX_BYTES} bytes without surrounding "
                                   "whitespace or control characters")


@dataclass(frozen=True)
class TaskIdentity:
    """Task family and semantic version: binds reward, targets, metric, verifier and artifact semantics."""
    name: str
    version: int = 1

    def __post_init__(self):
        ok = isinstance(self.name, str) and 0 < len(self.name) <= 64 and \
            all(c.islower() or c.isdigit() or c in "-_." for c in self.name)
        if not ok:
            raise InvalidConfiguration("task name must be 1..=64 characters of [a-z0-9._-]")
        if not isinstance(self.version, int) or self.version < 1:
            raise InvalidConfiguration("task version must be >= 1")


@dataclass(frozen=True)
class MetricContract:
    """The final metric, frozen into the launch before training starts."""
    name: str
    unit: str
    direction: str
    baseline: float
    minimum_material_improvement: float

    def validate(self) -> None:
        _label("metric name", self.name)
        _label("metric unit", self.unit)
        if self.direction not in (HIGHER_IS_BETTER, LOWER_IS_BETTER):
            raise InvalidFinalEvidence(f"metric direction must be {HIGHER_IS_BETTER} or {LOWER_IS_BETTER}")
        if not (math.isfinite(self.baseline) and math.isfinite(self.minimum_material_improvement)) \
                or self.minimum_material_improvement < 0:
            raise InvalidFinalEvidence("metric baseline and non-negative materiality margin must be finite")


@dataclass(frozen=True)
class MetricReport:
    """A candidate's measured final metric beside the contract it was measured under."""
    name: str
    unit: str
    direction: str
    baseline: float
    candidate: float
    minimum_material_improvement: float

    @staticmethod
    def of(contract: MetricContract, candidate: float) -> "MetricReport":
        return MetricReport(contract.name, contract.unit, contract.direction, contract.baseline, float(candidate),
                            contract.minimum_material_improvement)

    def directional_improvement(self) -> float:
        return self.candidate - self.baseline if self.direction == HIGHER_IS_BETTER else self.baseline - self.candidate

    def is_material_win(self) -> bool:
        return self.directional_improvement() > self.minimum_material_improvement

    def validate_against(self, c: MetricContract) -> None:
        MetricContract(self.name, self.unit, self.direction, self.baseline, self.minimum_material_improvement).validate()
        if not math.isfinite(self.candidate) or not math.isfinite(self.directional_improvement()):
            raise InvalidFinalEvidence("candidate metric and its directional improvement must be finite")
        same = (self.name, self.unit, self.direction) == (c.name, c.unit, c.direction) and \
            self.baseline.hex() == float(c.baseline).hex() and \
            float(self.minimum_material_improvement).hex() == float(c.minimum_material_improvement).hex()
        if not same:
            raise InvalidFinalEvidence("candidate metric does not exactly match the launch-frozen metric contract")


def metric_is_stronger(a: MetricReport, b: MetricReport) -> bool:
    """Strictly stronger in the contract's direction (exact ties keep the incumbent)."""
    return a.directional_improvement() > b.directional_improvement()


@dataclass
class FinalEvidence:
    """What a task verifier measured for one candidate."""
    held_out_correct: bool
    metric: MetricReport
    artifact: Any                      # JSON-serialisable payload, written only after acceptance
    verification_evidence: Any         # JSON-serialisable verifier evidence, kept beside the artifact


@dataclass
class CandidateVerification:
    """Either ``rejected(reason)`` (a normal invalid candidate) or ``measured(evidence)``."""
    evidence: Optional[FinalEvidence] = None
    reason: str = ""

    @staticmethod
    def rejected(reason: str) -> "CandidateVerification":
        return CandidateVerification(None, reason)

    @staticmethod
    def measured(evidence: FinalEvidence) -> "CandidateVerification":
        return CandidateVerification(evidence, "")


@dataclass(frozen=True)
class Candidate:
    """Read-only view of one authenticated candidate handed to ``verify_candidate``."""
    completion: str
    search_reward: float
    step: int
    prompt_index: int
    group_index: int
    provenance_sha256: str


@dataclass
class DiscoveryTask:
    """A task: identity, typed samples, the search reward and (optionally) the final verifier.

    Without ``verify_candidate`` the run stops after training and evaluation and reports the ranked
    candidates; with it (and a ``metric_contract``) the run ends in verified / no-win / preempted."""
    name: str
    samples: Sequence[Sample]
    reward_fn: RewardFn
    eval_samples: Sequence[Sample] = ()
    version: int = 1
    metric_contract: Optional[MetricContract] = None
    verify_candidate: Optional[Callable[[Candidate], CandidateVerification]] = None

    def identity(self) -> TaskIdentity:
        return TaskIdentity(self.name, self.version)


@dataclass
class DiscoveryConfig:
    model_dir: str
    out_dir: str = "runs"
    device: str = "cpu"
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    policy: PolicyCfg = field(default_factory=PolicyCfg)
    candidate_top_k: int = 4
    allow_dirty: bool = True
    artifact_output: Optional[str] = None
    preemption_flag: Any = None        # threading.Event

    def validate(self) -> None:
        if not self.model_dir:
            raise InvalidConfiguration("checkpoint_dir must not be empty")
        if not self.out_dir:
            raise InvalidConfiguration("runs_root must not be empty")
        if self.candidate_top_k < 1:
            raise InvalidConfiguration("candidate_top_k must be >= 1")
        t = self.trainer
        if t.steps < 1:
            raise InvalidConfiguration("steps must be >= 1")
        if t.group_size < 2:
            raise InvalidConfiguration("group_size must be >= 2 for world-one GRPO")
        if t.max_new_tokens < 1:
            raise InvalidConfiguration("max_new_tokens must be >= 1")
        if not math.isfinite(t.temperature) or t.temperature <= 0:
            raise InvalidConfiguration("temperature must be finite and > 0")
        if not math.isfinite(t.lr) or t.lr <= 0:
            raise InvalidConfiguration("learning_rate must be finite and > 0")
        if self.artifact_output is not None:
            if not self.artifact_output:
                raise InvalidConfiguration("artifact_output must not be empty")
            runs, art = os.path.abspath(self.out_dir), os.path.abspath(self.artifact_output)
            if runs == art or runs.startswith(art + os.sep):
                raise InvalidConfiguration(f"artifact_output {self.artifact_output} must not equal or contain "
                                           f"runs_root {self.out_dir}")

    class Builder:
        def __init__(self, model_dir: str):
            self._c = DiscoveryConfig(model_dir)

        def out_dir(self, p):
            self._c.out_dir = p
            return self

        def artifact_output(self, p):
            self._c.artifact_output = p
            return self

        def device(self, d):
            self._c.device = d
            return self

        def trainer(self, t: TrainerConfig):
            self._c.trainer = t
            return self

        def lora(self, rank: int, alpha: float):
            self._c.policy.lora_rank, self._c.policy.lora_alpha = rank, alpha
            return self

        def candidate_top_k(self, k: int):
            self._c.candidate_top_k = k
            return self

        def preemption_flag(self, flag):
            self._c.preemption_flag = flag
            return self

        def build(self) -> "DiscoveryConfig":
            self._c.validate()
            self._c.trainer.candidate_log_top_k = self._c.candidate_top_k
            self._c.trainer.validate()
            return self._c


# ------------------------------------------------------------------ outcomes
NO_WIN_CANDIDATES_REJECTED = "candidates_rejected"
NO_WIN_HELD_OUT_INCORRECT = "held_out_incorrect"
NO_WIN_NO_MATERIAL_METRIC_WIN = "no_material_metric_win"


@dataclass
class VerifiedArtifact:
    output: str
    manifest_path: str
    payload_path: str
    candidate_path: str
    verification_evidence_path: str
    task_identity: TaskIdentity
    candidate_sha256: str
    metric: MetricReport


@dataclass
class NoWinReport:
    run_dir: str
    candidates_checked: int
    reason: str
    detail: str


@dataclass
class DiscoveryOutcome:
    """``kind``: ``verified`` (artifact published), ``no_win``, ``preempted``, or ``ranked`` when the
    task carries no final verifier."""
    run_dir: str
    stop: str
    steps_run: int
    health_verdict: str
    best: list                     # CandidateRecord, best first
    eval_improvement: Optional[float]
    kind: str = "ranked"
    artifact: Optional[VerifiedArtifact] = None
    no_win: Optional[NoWinReport] = None

    def to_json(self):
        d = {"run_dir": self.run_dir, "stop": self.stop, "steps_run": self.steps_run, "kind": self.kind,
             "health_verdict": self.health_verdict, "eval_improvement": self.eval_improvement,
             "best": [{"reward": c.reward, "step": c.step, "completion": c.completion} for c in self.best]}
        if self.artifact is not None:
            d["artifact"] = {"output": self.artifact.output, "candidate_sha256": self.artifact.candidate_sha256,
                             "metric": asdict(self.artifact.metric)}
        if self.no_win is not None:
            d["no_win"] = asdict(self.no_win)
        return d


# ------------------------------------------------------------------ selection and publication
def select_winner(task: DiscoveryTask, contract: MetricContract, candidates: Sequence) -> tuple:
    """Check every authenticated candidate (already ranked best search reward first).

    Returns ``(index, evidence)`` of the strongest material winner, or ``(None, (checked, reason, detail))``."""
    contract.validate()
    checked, saw_measured = 0, False
    reason, detail = NO_WIN_CANDIDATES_REJECTED, "every candidate was rejected by the final verifier"
    best_i, best_ev = None, None
    for i, rec in enumerate(candidates):
        checked += 1
        view = Candidate(rec.completion, float(rec.reward), int(rec.step), int(rec.prompt_index), int(rec.group_index),
                         rec.record_sha256 or rec.digest())
        try:
            decision = task.verify_candidate(view)
        except TaskVerificationError:
            raise
        except Exception as e:  # noqa: BLE001 - a crashing verifier is an operational failure, not a rejection
            raise TaskVerificationError(f"final verifier failed on candidate {i}: {e!r}") from e
        if not isinstance(decision, CandidateVerification):
            raise TaskVerificationError("verify_candidate must return a CandidateVerification")
        ev = decision.evidence
        if ev is None:
            if not saw_measured:
                reason = NO_WIN_CANDIDATES_REJECTED
                detail = decision.reason if decision.reason.strip() else "candidate rejected without task detail"
            continue
        saw_measured = True
        ev.metric.validate_against(contract)
        if not ev.held_out_correct:
            reason, detail = NO_WIN_HELD_OUT_INCORRECT, "final verifier did not prove task-semantic held-out correctness"
            continue
        if not ev.metric.is_material_win():
            reason = NO_WIN_NO_MATERIAL_METRIC_WIN
            detail = (f"directional improvement {ev.metric.directional_improvement()} did not strictly exceed "
                      f"materiality margin {ev.metric.minimum_material_improvement}")
            continue
        if best_ev is None or metric_is_stronger(ev.metric, best_ev.metric):
            best_i, best_ev = i, ev
    if best_ev is not None:
        return best_i, best_ev
    return None, (checked, reason, detail)


def _dump(obj) -> bytes:
    return json.dumps(obj, sort_keys=True, indent=2, allow_nan=False).encode() + b"\n"


def _write_new_synced(path: str, data: bytes) -> None:
    fd = os.open(path, os.O_WRONLY | os.O_CREAT | os.O_EXCL, 0o644)
    with os.fdopen(fd, "wb") as f:
        f.write(data)
        f.flush()
        os.fsync(f.fileno())


def publish_verified_artifact(output: str, task: TaskIdentity, run_id: str, launch_bytes: bytes,
                              held_out_bytes: bytes, candidate, evidence: FinalEvidence,
                              fault_hook: Optional[Callable[[str], None]] = None) -> VerifiedArtifact:
    """Write the accepted bundle next to its destination, manifest last, then rename it into place.
    ``output`` must not exist; a failure before the rename leaves nothing at ``output``."""
    if os.path.lexists(output):
        raise InvalidConfiguration(f"artifact output already exists: {output}")
    parent = os.path.dirname(os.path.abspath(output))
    os.makedirs(parent, exist_ok=True)
    stage = os.path.join(parent, f".tmp-{os.path.basename(output)}-{os.getpid():x}-{os.urandom(4).hex()}")
    os.mkdir(stage)
    cand_body = dict(candidate.body(), record_sha256=candidate.record_sha256, record_signature=candidate.record_signature)
    files = {
        "artifact.json": _dump(evidence.artifact),
        "launch.json": launch_bytes,
        "eval-report.json": held_out_bytes,
        "candidate.json": _dump(cand_body),
        "verifier-evidence.json": _dump({"contract": VERIFIER_EVIDENCE_CONTRACT, "held_out_correct": True,
                                         "metric": asdict(evidence.metric),
                                         "evidence": evidence.verification_evidence}),
    }
    try:
        for name in ARTIFACT_FILES:
            _write_new_synced(os.path.join(stage, name), files[name])
        if fault_hook is not None:
            fault_hook("before_manifest")
        launch = json.loads(launch_bytes)
        manifest = {
            "contract": ARTIFACT_CONTRACT, "task": asdict(task), "run_id": run_id,
            "launch_sha256": launch.get("launch_sha256"), "candidate_public_key": launch.get("candidate_public_key"),
            "candidate_sha256": candidate.record_sha256 or candidate.digest(), "metric": asdict(evidence.metric),
            "files": {n: {"len": len(files[n]), "sha256": hashlib.sha256(files[n]).hexdigest()} for n in ARTIFACT_FILES},
        }
        _write_new_synced(os.path.join(stage, ARTIFACT_MANIFEST_FILE), _dump(manifest))
        fd = os.open(stage, os.O_RDONLY)
        try:
            os.fsync(fd)
        finally:
            os.close(fd)
        if os.path.lexists(output):
            raise InvalidConfiguration(f"artifact output already exists: {output}")
        os.rename(stage, output)
    except BaseException:
        for name in os.listdir(stage):
            os.unlink(os.path.join(stage, name))
        os.rmdir(stage)
        raise
    return VerifiedArtifact(output, os.path.join(output, ARTIFACT_MANIFEST_FILE), os.path.join(output, "artifact.json"),
                            os.path.join(output, "candidate.json"), os.path.join(output, "verifier-evidence.json"),
                            task, manifest["candidate_sha256"], evidence.metric)


def verify_artifact_bundle(output: str) -> dict:
    """Re-check a published bundle: contract tag, every file's length and SHA-256."""
    try:
        man = json.load(open(os.path.join(output, ARTIFACT_MANIFEST_FILE)))
    except (OSError, json.JSONDecodeError) as e:
        raise DiscoveryError(f"artifact bundle {output} has no readable manifest: {e}") from e
    if man.get("contract") != ARTIFACT_CONTRACT:
        raise DiscoveryError(f"artifact bundle {output} has contract {man.get('contract')!r}")
    if sorted(man.get("files", {})) != sorted(ARTIFACT_FILES):
        raise DiscoveryError("artifact manifest does not list exactly the bundle's files")
    for name, ent in man["files"].items():
        data = open(os.path.join(output, name), "rb").read()
        if len(data) != ent["len"] or hashlib.sha256(data).hexdigest() != ent["sha256"]:
            raise DiscoveryError(f"{name} of {output} does not match the manifest")
    return man


class Discovery:
    def __init__(self, task: DiscoveryTask, config: DiscoveryConfig, tokenizer=None, model_and_identity=None):
        self.task, self.config, self.tokenizer, self.model_and_identity = task, config, tokenizer, model_and_identity

    def _validate_before_load(self) -> None:
        c, t = self.config, self.task
        c.validate()
        t.identity()
        if not t.samples:
            raise InvalidConfiguration("discovery requires at least one training sample")
        if t.verify_candidate is not None:
            if t.metric_contract is None:
                raise InvalidConfiguration("a task with a final verifier must carry a metric contract")
            t.metric_contract.validate()
            if not t.eval_samples:
                raise InvalidConfiguration("discovery requires at least one task-semantic held-out sample")
            if c.artifact_output is None:
                raise InvalidConfiguration("a task with a final verifier needs an artifact_output")
            if os.path.lexists(c.artifact_output):
                raise InvalidConfiguration(f"artifact output already exists: {c.artifact_output}")

    def run(self) -> DiscoveryOutcome:
        import ferrl_b200.orchestration as orch
        from . import telemetry as T
        self._validate_before_load()
        c = self.config
        rc = RunConfig(task="countdown", model_dir=c.model_dir, device=c.device, out_dir=c.out_dir,
                       launch_authentication="signed", policy=c.policy, trainer=c.trainer)
        rc.trainer.candidate_log_top_k = c.candidate_top_k
        rc.eos_selection = "explicit" if rc.trainer.eos_token_id is not None else "disabled"
        task = self.task
        orig = orch.build_task
        orch.build_task = lambda _cfg: (list(task.samples), list(task.eval_samples), task.reward_fn)
        try:
            out: TrainOutcome = run_cli_train_setup(rc, allow_dirty=c.allow_dirty, tokenizer=self.tokenizer,
                                                    model_and_identity=self.model_and_identity,
                                                    preemption_flag=c.preemption_flag)
        finally:
            orch.build_task = orig
        res = DiscoveryOutcome(out.run_dir, out.stop, out.steps_run, out.health.verdict,
                               out.candidates[:c.candidate_top_k],
                               None if out.eval_report is None else out.eval_report.improvement())
        if out.stop == "preempted":
            res.kind = "preempted"
        elif task.verify_candidate is not None:
            if out.eval_report is None:
                raise DiscoveryError("the engine returned no held-out evaluation (run health failed or no eval samples)")
            idx, ev = select_winner(task, task.metric_contract, out.candidates)
            if idx is None:
                checked, reason, detail = ev
                res.kind, res.no_win = "no_win", NoWinReport(out.run_dir, checked, reason, detail)
            else:
                launch_bytes = open(os.path.join(out.run_dir, T.RunDir.LAUNCH_FILE), "rb").read()
                held_out = _dump({"contract": HELD_OUT_REPORT_CONTRACT, "sample_count": len(task.eval_samples),
                                  "report": out.eval_report.to_json()})
                res.artifact = publish_verified_artifact(c.artifact_output, task.identity(), out.run_id, launch_bytes,
                                                         held_out, out.candidates[idx], ev)
                res.kind = "verified"
        tmp = os.path.join(out.run_dir, "discovery-outcome.json.tmp")       # written last
        with open(tmp, "w") as f:
            json.dump(res.to_json(), f, indent=2, sort_keys=True)
        os.rename(tmp, os.path.join(out.run_dir, "discovery-outcome.json"))
        return res
