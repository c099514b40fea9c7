"""Command line: ``python -m ferrl_b200.cli <verb> ...``.

Verbs (reference ``crates/ferrl/src/bin/ferrl.rs:116-131``):

    train             --config run.json                  GRPO/LoRA training run
    score             (trimul-score) score external completions with the TriMul verifier
    audit             (trimul-artifact) paired-block audit of a run's best candidate
    report            (runreport) summarise a run directory's metrics and health
    perf-gate         compare a candidate run's metrics stream against a baseline's
    trimul-baseline   time the reference kernel to pin ``trimul.baseline.ns``
    verifier-executor serve the dedicated-UID verifier socket

The reference verb names are accepted as aliases.  Multi-GPU launches use one
process per GPU (``torchrun`` or Slurm ``srun`` with ``FERRL_NCCL_RENDEZVOUS``);
the communicator is opened from the environment.
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _comm():
    from .comm import NcclConfig, SoloComm, TorchDistComm
    cfg = NcclConfig.from_env()
    return SoloComm() if cfg is None or cfg.world_size == 1 else TorchDistComm.bootstrap(cfg)


def cmd_train(args) -> int:
    from .config import ConfigError, RunConfig
    from .orchestration import run_cli_train_setup
    try:
        cfg = RunConfig.load(args.config)
    except ConfigError as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    comm = _comm()
    if comm.world_size > 1 and cfg.tensor_parallel.enabled and cfg.distributed.enabled:
        print("error: data-parallel and tensor-parallel launches cannot be combined", file=sys.stderr)
        return 2
    if cfg.tensor_parallel.enabled:
        cfg.tensor_parallel.rank, cfg.tensor_parallel.world_size = comm.rank, comm.world_size
    out = run_cli_train_setup(cfg, comm, allow_dirty=args.allow_dirty)
    if comm.rank == 0:
        if out.health.findings:
            print(out.health.render(), file=sys.stderr, end="")
        print(json.dumps({"run_dir": out.run_dir, "stop": out.stop, "steps": out.steps_run,
                          "health": out.health.verdict,
                          "eval_improvement": None if out.eval_report is None else out.eval_report.improvement(),
                          "candidates": len(out.candidates)}))
    return 0 if out.health.verdict != "fail" else 1


def _trimul_reward(cfg):
    from .orchestration import build_task
    return build_task(cfg)[2]


LLAMA_CPP_EOT = "[end of text]"


def normalize_completion(raw: str, mode: str) -> tuple:
    """``(text, changed)``.  ``llama-cpp``: drop the ``[end of text]`` marker llama.cpp's CLI appends
    (and the whitespace around it), leaving one trailing newline."""
    if mode == "llama-cpp":
        stripped = raw.rstrip()
        if stripped.endswith(LLAMA_CPP_EOT):
            text = stripped[:-len(LLAMA_CPP_EOT)].rstrip() + "\n"
            return text, text != raw
    return raw, False


def read_verified_prompt_copy(path: str) -> bytes:
    """The prompt copy of a run directory, checked against the ``prompt.sha256`` beside it."""
    import hashlib
    data = open(path, "rb").read()
    hash_path = os.path.join(os.path.dirname(os.path.abspath(path)), "prompt.sha256")
    try:
        expected = (open(hash_path).read().split() or [""])[0]
    except OSError as e:
        raise ValueError(f"read {hash_path}: {e}") from e
    actual = hashlib.sha256(data).hexdigest()
    if expected != actual:
        raise ValueError(f"prompt copy hash mismatch: {hash_path} records {expected or '<empty>'}, but {path} "
                         f"hashes to {actual}")
    return data


def cmd_score(args) -> int:
    """Score external TriMul completions once with the shaped reward, on hidden cases re-keyed with
    ``--score-secret-seed`` (which must differ from the training seed)."""
    import hashlib
    from .config import RunConfig
    from .rewards.trimul import TRIMUL_CASE_SEED_MAX
    cfg = RunConfig.load(args.config)
    if cfg.task != "trimul":
        print("error: trimul-score requires a config with task \"trimul\"", file=sys.stderr)
        return 2
    if not 0 <= args.score_secret_seed <= TRIMUL_CASE_SEED_MAX:
        print(f"error: trimul-score requires --score-secret-seed between 0 and {TRIMUL_CASE_SEED_MAX}", file=sys.stderr)
        return 2
    if args.score_secret_seed == int(cfg.trimul.get("secret_seed", 0)):
        print("error: trimul-score requires --score-secret-seed to differ from trimul.secret_seed", file=sys.stderr)
        return 2
    try:
        prompt = read_verified_prompt_copy(args.prompt_copy)
    except (OSError, ValueError) as e:
        print(f"error: {e}", file=sys.stderr)
        return 2
    comps = []
    for p in args.completion or []:
        comps.append({"completion": open(p, encoding="utf-8").read(), "source_id": p})
    for p in args.completions_jsonl or []:
        for i, line in enumerate(open(p, encoding="utf-8")):
            if line.strip():
                d = json.loads(line)
                if not isinstance(d.get("completion"), str):
                    print(f"error: {p}:{i} has no completion string", file=sys.stderr)
                    return 2
                d.setdefault("source_id", f"{p}:{i}")
                comps.append(d)
    if not comps:
        print("error: trimul-score requires at least one --completion or --completions-jsonl row", file=sys.stderr)
        return 2
    if os.path.lexists(args.out):
        print(f"error: {args.out} already exists; scores are never overwritten", file=sys.stderr)
        return 2
    normalized = [normalize_completion(c["completion"], args.completion_normalization) for c in comps]
    reward = _trimul_reward(cfg).with_secret_seed(args.score_secret_seed)
    outs = reward.reward_group_detailed(None, [t for t, _ in normalized])
    if len(outs) != len(comps):
        print(f"error: trimul scoring returned {len(outs)} outcomes for {len(comps)} completions", file=sys.stderr)
        return 1
    config_sha = hashlib.sha256(open(args.config, "rb").read()).hexdigest()
    diagnostics: dict = {}
    with open(args.out, "x", encoding="utf-8") as f:
        for i, (c, (text, changed), o) in enumerate(zip(comps, normalized, outs)):
            if o.diagnostic:
                diagnostics[o.diagnostic] = diagnostics.get(o.diagnostic, 0) + 1
            meta = c.get("metadata")
            if args.completion_normalization != "none":
                meta = dict(meta or {}, completion_normalization={
                    "mode": args.completion_normalization, "changed": changed,
                    "raw_len_bytes": len(c["completion"].encode()),
                    "raw_sha256": hashlib.sha256(c["completion"].encode()).hexdigest()})
            f.write(json.dumps({
                "task": "trimul", "score_scheme": reward.profile.scheme, "run_id": args.run_id,
                "step": c.get("step", args.step), "rank": c.get("rank", args.rank),
                "world_size": c.get("world_size", args.world_size),
                "prompt_index": c.get("prompt_index", args.prompt_index), "group_index": c.get("group_index", i),
                "reward": o.reward, "reward_diagnostic": o.diagnostic, "reward_metadata": o.metadata,
                "input_metadata": meta, "input_reward_metadata": c.get("reward_metadata"),
                "completion_len_tokens": c.get("completion_len_tokens"), "completion_len_bytes": len(text.encode()),
                "completion": text,
                "external_score": {"model_family": args.model_family, "checkpoint": args.checkpoint,
                                   "tokenizer": args.tokenizer, "source_label": args.source_label,
                                   "source_id": c["source_id"], "source_index": i,
                                   "score_secret_seed": args.score_secret_seed, "used_training_secret_seed": False,
                                   "prompt_sha256": hashlib.sha256(prompt).hexdigest(), "config_sha256": config_sha},
            }, sort_keys=True) + "\n")
    print(json.dumps({"scored": len(comps), "positive": sum(1 for o in outs if o.reward > 0),
                      "best": max(o.reward for o in outs), "diagnostics": diagnostics, "out": args.out}, sort_keys=True))
    return 0


SOURCE_INSPECTION_RESULTS = ("clean", "suspicious", "not_performed")


def cmd_audit(args) -> int:
    """Extract one launch-bound candidate row (``--candidate-sha256``, default: the best-ranked one)
    and audit it: correctness on re-keyed secret cases, then 11 paired blocks in which the
    packaged baseline submission and the candidate are both run, in the block's scheduled order,
    on the one device named by ``--audit-cuda-visible-device``."""
    from .artifact import ArtifactError, publish_trimul_artifact
    from .config import RunConfig
    from .orchestration import OrchestrationError, load_and_rank_candidates
    from .rewards.trimul import default_eval_dir, extract_submission
    if os.path.lexists(args.out):
        print(f"error: {args.out} already exists; an audit claims a new output directory", file=sys.stderr)
        return 2
    try:
        cands = load_and_rank_candidates(args.run_dir)
    except OrchestrationError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    if not cands:
        print("error: the run has no authenticated candidates", file=sys.stderr)
        return 1
    if args.candidate_sha256:
        match = [c for c in cands if c.record_sha256 == args.candidate_sha256]
        if not match:
            print(f"error: no candidate row with record_sha256 {args.candidate_sha256}", file=sys.stderr)
            return 1
        best = match[0]
    else:
        best = cands[0]
    cfg = RunConfig.from_json(json.load(open(os.path.join(args.run_dir, "config.json"))))
    if args.audit_verifier_executor_socket:
        cfg.trimul["verifier_isolation_tier"] = "dedicated_uid_service_v1"
        cfg.trimul["verifier_executor_socket"] = args.audit_verifier_executor_socket
    if args.audit_cuda_visible_device is not None:
        os.environ["CUDA_VISIBLE_DEVICES"] = args.audit_cuda_visible_device
    reward = _trimul_reward(cfg)
    src = extract_submission(best.completion, reward.extract_mode)
    if src is None:
        print("error: the candidate contains no extractable submission", file=sys.stderr)
        return 1
    ref_src = open(os.path.join(cfg.trimul.get("eval_dir") or default_eval_dir(), "reference_submission.py"),
                   encoding="utf-8").read()

    def verify(source, seed):
        return reward.with_secret_seed(seed).verify_submission(source).correct

    def time_pair(source, first):
        order = [("reference", ref_src), ("candidate", source)]
        if first == "candidate":
            order.reverse()
        ns = {}
        for name, code in order:
            ev = reward.verify_submission(code)
            ns[name] = ev.geomean_ns if (ev.correct and ev.geomean_ns and not ev.implausible()) else float("nan")
        return ns["reference"], ns["candidate"]
    try:
        man = publish_trimul_artifact(args.run_dir, args.out, src, best.reward, verify, time_pair,
                                      run_health=args.run_health, source_inspection=args.source_inspection,
                                      source_inspection_notes=args.source_inspection_notes)
    except ArtifactError as e:
        print(f"error: {e}", file=sys.stderr)
        return 1
    print(json.dumps({"accepted": man.accepted, "wins": man.decision["observed_material_wins"],
                      "candidate_record_sha256": best.record_sha256, "out": args.out}))
    return 0 if man.accepted else 1


def cmd_report(args) -> int:
    """One-glance summary of a finished run (a run directory or a ``metrics.jsonl``).  ``--config``
    applies that run configuration's ``run_health`` policy; ``--strict`` exits 2 when the summary
    flags anomalies or the policy has findings (otherwise: 0 healthy, 1 not)."""
    from . import telemetry as T
    from .run_health import evaluate_run_health
    if os.path.isfile(args.run_dir):
        run_id, rows, cands = os.path.basename(os.path.dirname(os.path.abspath(args.run_dir))), T.read_metrics(args.run_dir), None
    else:
        rd = T.RunDir.open(args.run_dir)
        run_id = rd.run_id
        rows = T.read_metrics(rd.metrics_path) if os.path.exists(rd.metrics_path) else []
        cands = T.read_candidates(rd.candidates_path) if os.path.exists(rd.candidates_path) else None
    s = T.summarize(rows)
    out = {"run_id": run_id, "steps": s.steps, "reward_first": s.reward_first, "reward_last": s.reward_last,
           "reward_best": s.reward_best, "mean_step_secs": s.mean_step_secs,
           "mean_tokens_per_sec": s.mean_tokens_per_sec, "final_grad_norm": s.final_grad_norm,
           "peak_mem_bytes": s.peak_mem_bytes, "healthy": s.healthy(), "anomalies": [str(a) for a in s.anomalies]}
    policy = None
    if args.config:
        from .config import ConfigError, RunConfig
        try:
            cfg = RunConfig.load(args.config)
        except ConfigError as e:
            print(f"error: {e}", file=sys.stderr)
            return 2
        policy = evaluate_run_health(rows, cfg.run_health, cands, group_size=cfg.trainer.group_size,
                                     prompt_groups_per_step=cfg.trainer.grad_accum_steps * cfg.trainer.prompts_per_item)
        out["run_health"] = {"verdict": policy.verdict,
                             "findings": [{"rule": f.rule, "action": f.action, "message": f.message} for f in policy.findings]}
    if args.json:
        print(json.dumps(out, sort_keys=True))
    else:
        print(f"run {run_id}: {s.steps} steps, reward {s.reward_first:.4f} -> {s.reward_last:.4f} "
              f"(best {s.reward_best:.4f}), {s.mean_step_secs:.3f} s/step, {s.mean_tokens_per_sec:.1f} tok/s")
        for a in s.anomalies:
            print(f"  anomaly: {a}")
        if s.healthy():
            print("  healthy")
        if policy is not None:
            print(policy.render(), end="")
    flagged = bool(s.anomalies) or (policy is not None and bool(policy.findings))
    if args.strict and flagged:
        return 2
    return 0 if s.healthy() and not (policy is not None and policy.is_fail()) else 1


def _metrics_of(path: str):
    from . import telemetry as T
    p = path if os.path.isfile(path) else os.path.join(path, T.RunDir.METRICS_FILE)
    return T.read_metrics(p)


def cmd_perf_gate(args) -> int:
    """Compare two finished runs; several ``--baseline`` / ``--candidate`` paths are the ranks of one
    data-parallel job and need ``--distributed-world-max`` (gate the job as a whole: slowest rank,
    largest peak) with ``--distributed-world-size`` equal to the number of paths given."""
    from . import telemetry as T
    ratio = 1.0 + args.max_step_secs_regression_pct / 100.0 if args.max_step_ratio is None else args.max_step_ratio
    budget = T.RegressionBudget(
        require_timing=not args.skip_step_time_check, require_cuda_memory=not (args.skip_memory_check or args.no_memory),
        allow_health_warnings=args.allow_health_warnings, warmup_steps=args.warmup_steps,
        min_positive_grad_steps=args.min_positive_grad_steps, max_mean_step_secs_ratio=ratio,
        max_mean_step_secs_abs_slack=args.step_secs_slack,
        max_cuda_peak_used_ratio=1.0 + args.max_peak_mem_regression_pct / 100.0,
        max_cuda_peak_used_abs_slack_bytes=args.peak_mem_slack_bytes,
        max_final_grad_norm_rel_drift=args.max_final_grad_norm_rel_drift)
    many = len(args.baseline) > 1 or len(args.candidate) > 1
    if many and not args.distributed_world_max:
        print("error: several --baseline/--candidate paths are the ranks of one job; pass --distributed-world-max",
              file=sys.stderr)
        return 2
    if args.distributed_world_max:
        n = args.distributed_world_size
        if n is None or n != len(args.baseline) or n != len(args.candidate):
            print("error: --distributed-world-max needs --distributed-world-size equal to the number of --baseline "
                  "and of --candidate paths", file=sys.stderr)
            return 2
        rep = T.compare_world_max_metrics([_metrics_of(p) for p in args.baseline],
                                          [_metrics_of(p) for p in args.candidate], budget)
    else:
        rep = T.compare_metrics(_metrics_of(args.baseline[0]), _metrics_of(args.candidate[0]), budget)
    out = {"passed": rep.passed, "failures": rep.failures, "baseline_mean_step_secs": rep.baseline_mean_step_secs,
           "candidate_mean_step_secs": rep.candidate_mean_step_secs, "baseline_peak_bytes": rep.baseline_peak_bytes,
           "candidate_peak_bytes": rep.candidate_peak_bytes}
    if args.json:
        print(json.dumps(out, sort_keys=True))
    else:
        print(f"perf gate - {'PASS' if rep.passed else 'FAIL'}: step {rep.baseline_mean_step_secs:.4f} s -> "
              f"{rep.candidate_mean_step_secs:.4f} s, peak {rep.baseline_peak_bytes} B -> {rep.candidate_peak_bytes} B")
        for f in rep.failures:
            print(f"  {f}")
    return 0 if rep.passed else 1


def cmd_trimul_baseline(args) -> int:
    from .config import RunConfig
    cfg = RunConfig.load(args.config)
    reward = _trimul_reward(cfg)
    from .rewards.trimul import default_eval_dir
    ref_path = os.path.join(cfg.trimul.get("eval_dir") or default_eval_dir(), "reference_submission.py")
    ev = reward.verify_submission(open(ref_path, encoding="utf-8").read())
    print(json.dumps({"baseline_ns": ev.geomean_ns, "correct": ev.correct}))
    return 0 if ev.correct and ev.geomean_ns else 1


def cmd_verifier_executor(args) -> int:
    from .sandbox import ApptainerSandbox
    from .verifier_executor import serve_verifier_executor, validate_service_config
    validate_service_config(args.socket, args.work_root, args.client_uid, args.apptainer, args.socket_mode)
    os.makedirs(args.work_root, exist_ok=True)
    serve_verifier_executor(args.socket, ApptainerSandbox(args.apptainer), client_uid=args.client_uid,
                            socket_mode=args.socket_mode)
    return 0


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="ferrl-b200")
    sub = ap.add_subparsers(dest="verb", required=True)
    p = sub.add_parser("train")
    p.add_argument("--config", required=True)
    p.add_argument("--allow-dirty", action="store_true")
    p.set_defaults(fn=cmd_train)
    p = sub.add_parser("score", aliases=["trimul-score"])
    p.add_argument("--config", required=True)
    p.add_argument("--prompt-copy", required=True, help="prompt.txt of a run directory (prompt.sha256 beside it)")
    p.add_argument("--completion", action="append")
    p.add_argument("--completions-jsonl", action="append")
    p.add_argument("--completion-normalization", choices=["none", "llama-cpp"], default="none")
    p.add_argument("--out", required=True)
    p.add_argument("--score-secret-seed", type=int, required=True)
    p.add_argument("--run-id", default="external-rollout")
    p.add_argument("--source-label", default="external")
    p.add_argument("--step", type=int, default=0)
    p.add_argument("--prompt-index", type=int, default=0)
    p.add_argument("--rank", type=int, default=0)
    p.add_argument("--world-size", type=int, default=1)
    p.add_argument("--model-family", default="external")
    p.add_argument("--checkpoint")
    p.add_argument("--tokenizer")
    p.set_defaults(fn=cmd_score)
    p = sub.add_parser("audit", aliases=["trimul-artifact"])
    p.add_argument("--run-dir", required=True)
    p.add_argument("--candidate-sha256", help="record_sha256 of one row of candidates.jsonl (default: the best-ranked row)")
    p.add_argument("--out", required=True)
    p.add_argument("--audit-verifier-executor-socket")
    p.add_argument("--audit-cuda-visible-device")
    p.add_argument("--run-health", default="ok")
    p.add_argument("--source-inspection", default="not_performed", choices=SOURCE_INSPECTION_RESULTS)
    p.add_argument("--source-inspection-notes", default="")
    p.set_defaults(fn=cmd_audit)
    p = sub.add_parser("report", aliases=["runreport"])
    p.add_argument("run_dir", help="a run directory or a metrics.jsonl file")
    p.add_argument("--config", help="run configuration whose run_health policy is applied")
    p.add_argument("--json", action="store_true")
    p.add_argument("--strict", action="store_true", help="exit 2 on any anomaly or policy finding")
    p.set_defaults(fn=cmd_report)
    p = sub.add_parser("perf-gate")
    p.add_argument("--baseline", required=True, action="append")
    p.add_argument("--candidate", required=True, action="append")
    p.add_argument("--distributed-world-max", action="store_true")
    p.add_argument("--distributed-world-size", type=int)
    p.add_argument("--max-peak-mem-regression-pct", type=float, default=0.0)
    p.add_argument("--peak-mem-slack-bytes", type=int, default=64 * 1024 * 1024)
    p.add_argument("--max-step-secs-regression-pct", type=float, default=10.0)
    p.add_argument("--step-secs-slack", type=float, default=0.0)
    p.add_argument("--min-positive-grad-steps", type=int, default=1)
    p.add_argument("--max-final-grad-norm-rel-drift", type=float)
    p.add_argument("--skip-memory-check", action="store_true")
    p.add_argument("--skip-step-time-check", action="store_true")
    p.add_argument("--allow-health-warnings", action="store_true")
    p.add_argument("--json", action="store_true")
    p.add_argument("--max-step-ratio", type=float, help="alternative to --max-step-secs-regression-pct: a ratio")
    p.add_argument("--warmup-steps", type=int, default=0)
    p.add_argument("--no-memory", action="store_true", help="same as --skip-memory-check")
    p.set_defaults(fn=cmd_perf_gate)
    p = sub.add_parser("trimul-baseline")
    p.add_argument("--config", required=True)
    p.set_defaults(fn=cmd_trimul_baseline)
    p = sub.add_parser("verifier-executor")
    p.add_argument("--socket", default="/run/ferrl/verifier-executor.sock")
    p.add_argument("--work-root", default="/var/lib/ferrl/verifier-executor")
    p.add_argument("--apptainer", default="/usr/bin/apptainer")
    p.add_argument("--client-uid", type=int, required=True, help="the only UID whose requests are served")
    p.add_argument("--socket-mode", type=lambda v: int(v, 8), default=0o660)
    p.set_defaults(fn=cmd_verifier_executor)
    args = ap.parse_args(argv)
    return args.fn(args)


if __name__ == "__main__":
    sys.exit(main())
