"""Run orchestration: from a validated ``RunConfig`` to a finished, provenance-bound run.

Reference ``crates/ferrl/src/orchestration.rs``: launch manifest types
``:82-470``; ``run_cli_train_setup`` ``:1094-1316`` (config / commit consensus,
synchronised run id ``<task>-<unix secs>[-rankN]``, device preflight, task data);
engine stages setup -> preflight -> launch -> train -> health -> eval ->
candidates ``:1885-1896``; health policy ``:3202-3970``; authenticated candidate
loading and ranking ``:4020-4560``.

Stages here:

1. ``setup``      build identity + config consensus, run id, device preflight,
                  task data, policy load, EOS resolution and consensus.
2. ``launch``     ``LaunchManifest`` (digests of config, policy, tokenizer,
                  prompts; build identity; candidate signing key) ->
                  ``RunDir.create`` -> immutable ``launch.json`` / ``config.json``.
3. ``train``      ``Trainer.resume_latest`` then ``Trainer.train``.
4. ``health``     ``telemetry.summarize`` + the configured run-health rules;
                  a ``fail`` finding blocks publication.
5. ``eval``       held-out base-vs-adapter evaluation -> ``eval-report.json``.
6. ``candidates`` verify signatures against ``launch.json`` and rank.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import os
import time
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

import torch

from . import telemetry as T
from .build_identity import BuildIdentity, require_clean, source_identity
from .checkpoint import CheckpointBinding
from .comm import Comm, SoloComm
from .config import RunConfig, canonical_digest
from .eval import EvalReport, evaluate
from .hf import resolve_eos, validate_resolved_eos_consensus
from .lm_policy import LmPolicy
from .models.loader import LoaderOpts, load_auto_policy
from .models.lora import BaseQuantization, DenseLoraTargets, LoraSpec
from .policy import GenConfig
from .run_health import HealthFinding, HealthReport, evaluate_run_health  # noqa: F401
from .rewards import (CountdownConfig, CountdownProblem, CountdownReward, MathProblem, MathReward, Sample, build_prompt,
                      generate_dataset, math_prompt, read_jsonl, train_eval_split, train_eval_split_by_key)
from .sampler import GrpoSampler
from .trainer import RunStop, Trainer


class OrchestrationError(RuntimeError):
    pass


@dataclass
class LaunchManifest:
    run_id: str
    task: str
    config_sha256: str
    policy_sha256: str
    tokenizer_sha256: str
    samples_sha256: str
    build: dict
    world_size: int
    topology: str
    candidate_public_key: Optional[str]
    launch_authentication: str
    created_unix: int
    evaluation_samples_sha256: Optional[str] = None

    def to_json(self) -> dict:
        return dataclasses.asdict(self)

    def digest(self) -> str:
        return canonical_digest(self.to_json(), b"ferrl-b200/launch-manifest/v1")


def exact_execution_samples(samples) -> bytes:
    """The ordered samples as the JSON bytes whose SHA-256 the ranks must agree on.  The bytes must survive a parse
    and re-serialisation unchanged (no NaN, no value that only ``repr`` can express), so that a run can be rebuilt
    from them (reference: ``exact_execution_samples``, crates/ferrl/src/orchestration.rs:587-597)."""
    blob = ("[" + ",".join(s.key() for s in samples) + "]").encode()

    def reject(constant):
        raise OrchestrationError(f"samples contain {constant}, which strict JSON cannot carry")
    parsed = json.loads(blob.decode(), parse_constant=reject)
    if len(parsed) != len(samples) or any(set(p) != {"prompt", "target"} for p in parsed):
        raise OrchestrationError("samples do not round-trip through JSON")
    return blob


def preflight_prompt_tokenization(samples, kind: str, tokenizer) -> None:
    """A prompt that encodes to no tokens would silently become an empty model input
    (crates/ferrl/src/orchestration.rs:599-613)."""
    for index, sample in enumerate(samples):
        if len(tokenizer.encode(sample.prompt)) == 0:
            raise OrchestrationError(f"{kind} prompt at index {index} encoded to zero tokens with the loaded tokenizer")


def preflight_samples(train_samples, eval_samples, tokenizer, comm: Comm) -> tuple[str, str]:
    """The preflight stage of the engine (crates/ferrl/src/orchestration.rs:2027-2082): exact sample bytes and the
    tokenizer check run locally, a failure on any rank stops all of them together, then the ranks must agree on both
    digests.  Returns ``(training_sha256, evaluation_sha256)``."""
    def local():
        tb = exact_execution_samples(train_samples)
        eb = exact_execution_samples(eval_samples)
        preflight_prompt_tokenization(train_samples, "ordered training samples", tokenizer)
        preflight_prompt_tokenization(eval_samples, "ordered held-out samples", tokenizer)
        return hashlib.sha256(tb).hexdigest(), hashlib.sha256(eb).hexdigest()
    train_sha, eval_sha = comm.coordinate(local, "exact sample reconstruction and tokenizer preflight")
    comm.require_consensus(train_sha.encode(), "ordered training samples")
    comm.require_consensus(eval_sha.encode(), "ordered held-out samples")
    return train_sha, eval_sha


def synchronized_run_id(task: str, comm: Comm, suffix_rank: bool = False) -> str:
    """Rank 0's wall-clock second, shared with every rank."""
    stamp = comm.broadcast_bytes(str(int(time.time())).encode() if comm.rank == 0 else None, 0).decode() \
        if comm.world_size > 1 else str(int(time.time()))
    rid = f"{task}-{stamp}"
    return f"{rid}-rank{comm.rank}" if suffix_rank else rid


def build_task(cfg: RunConfig):
    """``(train_samples, eval_samples, reward_fn)`` for the configured task."""
    d = cfg.data
    if cfg.task == "countdown":
        if d.path:
            samples = read_jsonl(d.path, CountdownProblem.from_json)
        else:
            probs = generate_dataset(d.seed, d.train_n + d.eval_n, CountdownConfig())
            samples = [Sample(build_prompt(p), p) for p in probs]
        train, ev = train_eval_split_by_key(samples, d.eval_n, d.seed, lambda s: s.target.split_key())
        return train[:d.train_n] if d.train_n else train, ev, CountdownReward()
    if cfg.task == "math":
        if not d.path:
            raise OrchestrationError("the math task needs data.path (a JSONL of {prompt, target:{answer}})")
        from .rewards.math import math_split_key
        samples = read_jsonl(d.path, MathProblem.from_json)
        train, ev = train_eval_split_by_key(samples, d.eval_n, d.seed, math_split_key)
        return train[:d.train_n] if d.train_n else train, ev, MathReward()
    if cfg.task == "trimul":
        from .rewards.trimul import TrimulCase, TrimulReward, TrimulRewardProfile, default_eval_dir
        from .sandbox import ApptainerSandbox
        from .verifier_executor import SameUidApptainerSandbox, VerifierExecutorSandbox, VerifierIsolationTier
        t = dict(cfg.trimul)
        t.setdefault("eval_dir", default_eval_dir())
        for req in ("prompt_path", "image", "eval_dir"):
            if not t.get(req):
                raise OrchestrationError(f"trimul.{req} is required for the trimul task")
        prompt = open(t["prompt_path"], encoding="utf-8").read()
        tier = VerifierIsolationTier(t.get("verifier_isolation_tier", "same_uid_apptainer_v1"))
        if tier is VerifierIsolationTier.DEDICATED_UID_SERVICE_V1:
            sb = VerifierExecutorSandbox(t.get("verifier_executor_socket") or "/run/ferrl/verifier-executor.sock")
        else:
            sb = SameUidApptainerSandbox(ApptainerSandbox(t.get("verifier_apptainer_bin") or "apptainer"))
        cases = [TrimulCase(**c) for c in t.get("cases", [])] or [TrimulCase(32, 1, 16, 16, int(t.get("secret_seed", 0)))]
        reward = TrimulReward(sb, t["image"], t["eval_dir"], cases, scratch_root=t.get("scratch_root"),
                              profile=TrimulRewardProfile(**t["reward"]) if t.get("reward") else None,
                              baseline_ns=(t.get("baseline") or {}).get("ns"), wall_secs=float(t.get("wall_secs", 300)),
                              scratch_max_bytes=int(t.get("scratch_max_bytes", 2 << 30)),
                              parallelism=int(t.get("verifier_parallelism", 1)),
                              extract_mode=t.get("submission_extract_mode") or "final_fence")
        if t.get("held_out_secret_seed") is not None:
            # held-out evaluation runs on hidden inputs the policy was never scored on (ferrl.rs:1700-1712)
            import copy
            reward.held_out_reward = copy.copy(reward).with_secret_seed(int(t["held_out_secret_seed"]))
        samples = [Sample(prompt, {"trimul": i}) for i in range(max(d.train_n, 1))]
        return samples, samples[:max(d.eval_n, 0)], reward
    raise OrchestrationError(f"unknown task {cfg.task!r}")


_DTYPES = {"f32": torch.float32, "bf16": torch.bfloat16, "f16": torch.float16}


@dataclass
class TrainOutcome:
    run_dir: str
    run_id: str
    stop: str
    steps_run: int
    health: HealthReport
    eval_report: Optional[EvalReport]
    candidates: list


def run_cli_train_setup(cfg: RunConfig, comm: Optional[Comm] = None, *, allow_dirty: bool = False,
                        tokenizer=None, model_and_identity=None, preemption_flag=None,
                        heap_factory=None) -> TrainOutcome:
    """The whole ``train`` verb. ``tokenizer`` / ``model_and_identity`` may be injected (tests,
    synthetic runs); otherwise they are loaded from ``cfg.model_dir``.  ``preemption_flag`` is a
    ``threading.Event`` the caller sets to stop cooperatively after the step in flight.
    ``heap_factory(comm, device, wait_limit_s)`` replaces the symmetric heap (tests run the
    tensor-/expert-parallel wiring against a fake on CPU)."""
    comm = comm or SoloComm()
    T.init_tracing()
    ident = source_identity()
    require_clean(ident, allow_dirty)
    comm.require_consensus(cfg.digest().encode(), "run config")
    comm.require_consensus(ident.commit.encode(), "source commit")
    topology = "tp" if cfg.tensor_parallel.enabled else "dp"
    if comm.world_size > 1 and not (cfg.distributed.enabled or cfg.tensor_parallel.enabled):
        raise OrchestrationError("a multi-rank launch needs distributed.enabled or tensor_parallel.enabled")
    run_id = synchronized_run_id(cfg.task, comm)
    device = cfg.device
    if device.startswith("cuda"):
        from .preflight import check_device, guard_first_kernel
        idx = torch.cuda.current_device() if torch.cuda.is_available() else 0
        check_device(idx)
        guard_first_kernel()
        device = f"cuda:{idx}"
    # a rank that cannot build its task data stops all of them together (orchestration.rs:1202-1242)
    train_samples, eval_samples, reward_fn = comm.coordinate(lambda: build_task(cfg), f"{cfg.task} task setup")
    # ---- policy
    pc = cfg.policy
    # "all_linear" and a trailing "|gdn:<letters>" also select GatedDeltaNet projections of the hybrid families
    dense_targets, gdn_targets = pc.lora_targets, ""
    if dense_targets == "all_linear":
        dense_targets, gdn_targets = "industrial", "qzbao"
    elif "|gdn:" in dense_targets:
        dense_targets, gdn_targets = dense_targets.rsplit("|gdn:", 1)
        gdn_targets = "" if gdn_targets == "-" else gdn_targets
    lora = LoraSpec(pc.lora_rank, pc.lora_alpha, DenseLoraTargets.parse(dense_targets))
    ep_on = cfg.expert_parallel.enabled and comm.world_size > 1
    opts = LoaderOpts(dtype=_DTYPES[pc.base_dtype], device=device, lora=lora,
                      quantization=BaseQuantization(pc.base_quantization), remat=pc.activation_checkpointing,
                      tp=(cfg.tensor_parallel.rank, cfg.tensor_parallel.world_size) if cfg.tensor_parallel.enabled else None,
                      ep=(comm.rank, comm.world_size) if ep_on else None,
                      adapter_seed=pc.seed, gdn_targets=gdn_targets)
    # a rank that cannot load its share of the checkpoint stops all of them together instead of leaving the others
    # waiting in the first collective (orchestration.rs:1899-2025 coordinates every setup stage)
    model, pident = model_and_identity or comm.coordinate(lambda: load_auto_policy(cfg.model_dir, opts), "policy load")
    if cfg.tensor_parallel.enabled and cfg.tensor_parallel.sequence_parallel:
        if not hasattr(model, "sequence_parallel"):
            raise OrchestrationError("tensor_parallel.sequence_parallel is not supported by this model family")
        model.sequence_parallel = True
    def tokenizer_and_eos():
        tok = tokenizer
        if tok is None:
            from .tokenizer import HfTokenizer
            tok = HfTokenizer.from_file(cfg.model_dir)
        eos = cfg.trainer.eos_token_id
        if cfg.eos_selection != "disabled" and os.path.exists(os.path.join(cfg.model_dir, "config.json")):
            eos = resolve_eos(cfg.model_dir, cfg.eos_selection, eos, tok)
        return tok, eos
    tokenizer, cfg.trainer.eos_token_id = comm.coordinate(tokenizer_and_eos, "tokenizer load and EOS resolution")
    validate_resolved_eos_consensus(cfg.trainer.eos_token_id, comm)
    policy = LmPolicy(model, GrpoSampler(pc.seed, cfg.trainer.temperature), comm if topology == "tp" else None,
                      pad_token_id=cfg.trainer.eos_token_id or 0,
                      score_microbatch=cfg.trainer.backward_microbatch_size)
    parallel_rt = build_parallel_runtime(cfg, comm, device, model, topology, heap_factory=heap_factory)
    if ep_on:
        # dispatch and combine are collectives: every rank must issue the same number of model calls,
        # so no rank leaves the decode loop early and no rank skips a degenerate group on its own
        policy.early_exit_every = 0
    # ---- launch manifest + run dir
    samples_sha, eval_samples_sha = preflight_samples(train_samples, eval_samples, tokenizer, comm)
    launch_sha_seed = hashlib.sha256((run_id + cfg.digest()).encode()).digest()
    signer = None
    if cfg.launch_authentication == "signed":
        signer = T.CandidateSigner("", seed=None)
    manifest = LaunchManifest(run_id, cfg.task, cfg.digest(), pident.digest(), tokenizer.digest(), samples_sha,
                              ident.to_json(), comm.world_size, topology,
                              signer.public_key_hex if signer else None, cfg.launch_authentication, int(time.time()),
                              eval_samples_sha)
    if signer:
        signer.launch_sha256 = manifest.digest()
    del launch_sha_seed
    comm.require_consensus(json.dumps({k: v for k, v in manifest.to_json().items()
                                       if k not in ("candidate_public_key", "created_unix")}, sort_keys=True).encode(),
                           "launch manifest")
    def publish_run_dir():
        if comm.rank != 0:
            return None
        rd = T.RunDir.create(cfg.out_dir, run_id)
        rd.write_json_once(T.RunDir.LAUNCH_FILE, dict(manifest.to_json(), launch_sha256=manifest.digest()))
        rd.write_json_once(T.RunDir.CONFIG_FILE, cfg.to_json())
        return rd
    # the status exchange doubles as the barrier behind which the other ranks open the directory; a rank 0 that
    # cannot publish (duplicate run id, read-only root) stops every rank instead of leaving them at a barrier
    run_dir = comm.coordinate(publish_run_dir, "run directory publication") if comm.world_size > 1 else publish_run_dir()
    if run_dir is None:
        run_dir = T.RunDir(os.path.join(cfg.out_dir, run_id), run_id)
    binding = CheckpointBinding(pident.digest(), cfg.trainer.digest(), policy.lora_recipe())
    cand_writer = T.CandidateWriter(run_dir.candidates_path, signer) if comm.rank == 0 or topology == "dp" else None
    if cand_writer is not None and comm.rank != 0:
        cand_writer = T.CandidateWriter(run_dir.candidates_path + f".rank{comm.rank}", signer)
    fused = None
    if topology == "dp" and device.startswith("cuda"):
        from .parallel.dp import FusedDpStep
        fused = FusedDpStep.create(comm, policy.trainable_params(), torch.device(device))
    trainer = Trainer(policy, tokenizer, reward_fn, train_samples, cfg.trainer, comm=comm, topology=topology,
                      run_dir=run_dir, binding=binding, candidate_writer=cand_writer, fused_dp_step=fused,
                      parallel_runtime=parallel_rt, lockstep_model_calls=ep_on)
    if preemption_flag is not None:
        trainer.with_preemption_flag(preemption_flag)
    try:
        with T.run_span(comm.rank, comm.world_size):
            start = trainer.resume_latest()
            stop = trainer.train(start)
    except BaseException:
        if parallel_rt is not None:
            parallel_rt.close()
        raise
    # ---- health, eval, candidates (rank 0 owns publication)
    rows = trainer.history
    cands = T.read_candidates(run_dir.candidates_path) if comm.rank == 0 else []
    health = comm.coordinate(
        lambda: evaluate_run_health(rows, cfg.run_health, cands, group_size=cfg.trainer.group_size,
                                    prompt_groups_per_step=cfg.trainer.grad_accum_steps * cfg.trainer.prompts_per_item),
        "post-run health")
    # every rank holds its own metric rows (and rank 0 the candidate rows), so the verdicts may differ: a failure
    # anywhere stops the held-out evaluation everywhere, or the ranks would part ways in front of its collectives
    # (the reference aborts all ranks in lockstep on a failed post-run health check, orchestration.rs:2365-2410)
    health_failed = comm.all_reduce_scalar_sum(1.0 if health.verdict == "fail" else 0.0) > 0 if comm.world_size > 1 \
        else health.verdict == "fail"
    report = None
    if eval_samples and stop is RunStop.COMPLETED and not health_failed:
        gen = GenConfig(cfg.trainer.group_size, cfg.trainer.max_new_tokens, cfg.trainer.temperature,
                        cfg.trainer.eos_token_id)
        report = evaluate(policy, getattr(reward_fn, "held_out_reward", None) or reward_fn, tokenizer, eval_samples, gen)
        if comm.rank == 0:
            # published once, through a temporary file and a rename; an existing report is never replaced
            # (telemetry.rs: eval_report_publication_is_immutable)
            run_dir.write_json_once(T.RunDir.EVAL_REPORT_FILE, report.to_json())
    ranked = load_and_rank_candidates(run_dir.root, steps=cfg.trainer.steps, group_size=cfg.trainer.group_size,
                                      max_new_tokens=cfg.trainer.max_new_tokens, rank=0,
                                      world_size=comm.world_size) if comm.rank == 0 else []
    if parallel_rt is not None:
        parallel_rt.close()
    return TrainOutcome(run_dir.root, run_id, stop.value, len(rows), health, report, ranked)


def build_parallel_runtime(cfg: RunConfig, comm: Comm, device: str, model, topology: str, heap_factory=None):
    """The peer-memory data plane of a tensor- or expert-parallel launch (``None`` otherwise): a
    symmetric heap, the fused GEMM -> all-reduce and activation all-reduce registered for the
    tensor-parallel communicator, and the expert-parallel dispatch/combine runtime.  Buffer sizes come
    from the largest forward call the trainer makes (scoring micro-batch rows x longest sequence)."""
    tp_on = topology == "tp" and comm.world_size > 1
    ep_on = cfg.expert_parallel.enabled and comm.world_size > 1
    if not (tp_on or ep_on):
        return None
    from .parallel.runtime import ParallelRuntime
    spec = model.spec
    t = cfg.trainer
    rows_per_call = t.backward_microbatch_size if t.backward_microbatch_size > 0 else t.prompts_per_item * t.group_size
    tokens_cap = min(int(getattr(spec, "max_position_embeddings", 4096)), t.max_new_tokens + 2048)
    max_rows = min(max(rows_per_call, t.prompts_per_item * t.group_size) * tokens_cap, 1 << 16)
    ep = None
    if ep_on:
        moe = getattr(spec, "moe", None)
        if moe is None:
            raise OrchestrationError("expert_parallel.enabled needs a sparse-MoE policy")
        if moe.num_experts % comm.world_size:
            raise OrchestrationError(f"{moe.num_experts} experts do not split over {comm.world_size} ranks")
        ep = {"num_experts": moe.num_experts, "hidden": spec.hidden_size, "max_tokens": max_rows, "top_k": moe.top_k,
              "capacity_factor": cfg.expert_parallel.capacity_factor}
    return ParallelRuntime.create(comm, device, tensor_parallel=tp_on, hidden=spec.hidden_size, max_rows=max_rows,
                                  expert_parallel=ep, heap_factory=heap_factory,
                                  sequence_parallel=bool(tp_on and cfg.tensor_parallel.sequence_parallel))


def load_and_rank_candidates(run_root: str, require_signed: bool = True, *, steps: Optional[int] = None,
                             group_size: Optional[int] = None, max_new_tokens: Optional[int] = None,
                             rank: Optional[int] = None, world_size: Optional[int] = None,
                             require_complete: bool = False) -> list:
    """Authenticated candidates of a run, best reward first (ties: earlier step, lower prompt index,
    lower group index).  Every row must be newline-terminated, non-blank, signed for this launch
    and - when the launch bounds are given - lie inside them: ``step < steps``, ``group_index <
    group_size``, ``1 <= completion_len_tokens <= max_new_tokens``, the active rank/world; no two
    rows may claim one ``(step, prompt_index, group_index)``; ``require_complete`` demands exactly
    ``steps * group_size`` rows (reference orchestration.rs:4020-4180)."""
    try:
        launch = json.load(open(os.path.join(run_root, T.RunDir.LAUNCH_FILE)))
    except (OSError, json.JSONDecodeError) as e:
        raise OrchestrationError(f"cannot read launch.json of {run_root}: {e}") from e
    key, lsha = launch.get("candidate_public_key"), launch.get("launch_sha256")
    path = os.path.join(run_root, T.RunDir.CANDIDATES_FILE)
    if not os.path.exists(path):
        if require_complete:
            raise OrchestrationError("candidate ledger is missing")
        return []
    raw = open(path, "rb").read()
    if raw and not raw.endswith(b"\n"):
        raise OrchestrationError(f"candidate ledger {path} has an unterminated final row")
    try:
        text = raw.decode("utf-8")
    except UnicodeDecodeError as e:
        raise OrchestrationError(f"candidate ledger {path} is not UTF-8: {e}") from e
    out, seen = [], set()
    for n, line in enumerate(text.split("\n")[:-1] if text else [], 1):
        if not line.strip():
            raise OrchestrationError(f"candidate ledger {path} contains blank row {n}")
        try:
            rec = T.CandidateRecord(**json.loads(line))
        except (TypeError, json.JSONDecodeError) as e:
            raise OrchestrationError(f"candidate ledger {path} row {n} is malformed: {e}") from e
        if key:
            try:
                T.verify_candidate(rec, key, lsha)
            except ValueError as e:
                raise OrchestrationError(f"candidate ledger {path} row {n} failed launch authentication: {e}") from e
        elif require_signed and launch.get("launch_authentication") == "signed":
            raise OrchestrationError("run was launched as signed but carries no candidate key")
        if (rank is not None and rec.rank != rank) or (world_size is not None and rec.world_size != world_size):
            raise OrchestrationError(f"candidate ledger {path} row {n} rank/world disagree with active execution topology")
        if (steps is not None and rec.step >= steps) or (group_size is not None and rec.group_index >= group_size) \
                or rec.step < 0 or rec.group_index < 0:
            raise OrchestrationError(f"candidate ledger {path} row {n} coordinates exceed the launch config")
        if max_new_tokens is not None and not 1 <= rec.completion_len_tokens <= max_new_tokens:
            raise OrchestrationError(f"candidate ledger {path} row {n} completion length {rec.completion_len_tokens} "
                                     f"is outside the launch-bound range 1..={max_new_tokens}")
        pos = (rec.step, rec.prompt_index, rec.group_index)
        if pos in seen:
            raise OrchestrationError(f"candidate ledger {path} row {n} duplicates a training position")
        seen.add(pos)
        out.append(rec)
    if require_complete and steps is not None and group_size is not None and len(out) != steps * group_size:
        raise OrchestrationError(f"candidate ledger has {len(out)} rows, expected complete logging of {steps * group_size}")
    out.sort(key=lambda r: (-r.reward, r.step, r.prompt_index, r.group_index))
    return out
