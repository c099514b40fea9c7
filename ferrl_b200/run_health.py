"""Post-run health policy: typed rules over a run's metrics rows and candidate log.

Reference ``crates/ferrl/src/orchestration.rs:3202-3970``.  The ``run_health`` block of a run
configuration may carry

* ``reward_collapse``       ``{window, min, action}``  trailing-window mean reward below ``min``
* ``correctness_collapse``  ``{window, min, action}``  fraction of candidates the verifier marked
  correct over the trailing window below ``min`` (``min`` in [0, 1])
* ``dropped_rows``          ``{max, action}``          rows dropped over the whole run above ``max``
* ``grad_spike``            ``{factor, action}``       worst gradient norm above ``factor`` x the median
  of the positive finite norms
* ``telemetry_dark``        ``"warn" | "fail"``        no step captured behaviour log-probs, so the
  off-policy drift columns are empty
* ``source_dominance``      ``{max_fraction, action}`` one candidate source (``source_sha256`` of the
  reward metadata) supplies more than ``max_fraction`` of all candidates

Unknown keys are rejected; ``action`` is ``warn`` or ``fail`` (``stop`` is reserved for in-run gating
and refused); a window longer than ``trainer.steps`` is refused; the two candidate-based rules need
``trainer.candidate_log_top_k >= trainer.group_size`` so that every row of every group is logged,
and they report - instead of silently passing - when the candidate log is missing, empty, lacks a
step of the window, lacks full group coverage or carries no correctness metadata.  A non-finite
metric always fails the run.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Sequence

from .config import ConfigError

UNKNOWN_SOURCE = "__unknown_source__"
_RULE_KEYS = {
    "reward_collapse": {"window", "min", "action"},
    "correctness_collapse": {"window", "min", "action"},
    "dropped_rows": {"max", "action"},
    "grad_spike": {"factor", "action"},
    "source_dominance": {"max_fraction", "action"},
}


@dataclass
class HealthFinding:
    rule: str
    action: str     # warn | fail
    message: str


@dataclass
class HealthReport:
    verdict: str = "ok"    # ok | warn | fail
    findings: list = field(default_factory=list)

    def push(self, rule: str, action: str, message: str) -> None:
        self.findings.append(HealthFinding(rule, action, message))
        if action == "fail":
            self.verdict = "fail"
        elif self.verdict == "ok":
            self.verdict = "warn"

    def is_fail(self) -> bool:
        return self.verdict == "fail"

    def render(self) -> str:
        label = {"ok": "HEALTHY", "warn": "WARN", "fail": "FAIL"}[self.verdict]
        lines = [f"run health policy - {label}"]
        lines += [f"  {f.action.upper()} {f.rule}: {f.message}" for f in self.findings]
        return "\n".join(lines) + "\n"


def _action(label: str, a) -> str:
    if a == "stop":
        raise ConfigError(f"{label}.action = \"stop\" is reserved for future in-run gating; use \"warn\" or "
                          "\"fail\" for the post-run policy")
    if a not in ("warn", "fail"):
        raise ConfigError(f"{label}.action must be \"warn\" or \"fail\", got {a!r}")
    return a


def _num(label: str, v) -> float:
    if isinstance(v, bool) or not isinstance(v, (int, float)) or not math.isfinite(v):
        raise ConfigError(f"{label} must be finite")
    return float(v)


def validate_run_health(rules: dict, trainer) -> None:
    """Strict check of a ``run_health`` block against the trainer configuration it will judge."""
    if not isinstance(rules, dict):
        raise ConfigError("run_health must be a JSON object")
    unknown = set(rules) - set(_RULE_KEYS) - {"telemetry_dark"}
    if unknown:
        raise ConfigError(f"unknown field(s) in run_health: {sorted(unknown)}")
    for rule, keys in _RULE_KEYS.items():
        cfg = rules.get(rule)
        if cfg is None:
            continue
        label = f"run_health.{rule}"
        if not isinstance(cfg, dict) or set(cfg) != keys:
            raise ConfigError(f"{label} must be an object with exactly the fields {sorted(keys)}")
        _action(label, cfg["action"])
        if "window" in keys:
            w = cfg["window"]
            if isinstance(w, bool) or not isinstance(w, int) or w < 1:
                raise ConfigError(f"{label}.window must be >= 1")
            if w > trainer.steps:
                raise ConfigError(f"{label}.window ({w}) must be <= trainer.steps ({trainer.steps})")
            m = _num(f"{label}.min", cfg["min"])
            if rule == "correctness_collapse" and not 0.0 <= m <= 1.0:
                raise ConfigError(f"{label}.min must be in [0, 1]")
        if "max" in keys:
            mx = cfg["max"]
            if isinstance(mx, bool) or not isinstance(mx, int) or mx < 0:
                raise ConfigError(f"{label}.max must be a non-negative integer")
        if "factor" in keys and _num(f"{label}.factor", cfg["factor"]) <= 0:
            raise ConfigError(f"{label}.factor must be finite and > 0")
        if "max_fraction" in keys and not 0.0 <= _num(f"{label}.max_fraction", cfg["max_fraction"]) <= 1.0:
            raise ConfigError(f"{label}.max_fraction must be finite and in [0, 1]")
    if rules.get("telemetry_dark") is not None:
        _action("run_health.telemetry_dark", rules["telemetry_dark"])
    if (rules.get("correctness_collapse") or rules.get("source_dominance")) and \
            trainer.candidate_log_top_k < trainer.group_size:
        raise ConfigError("run_health correctness/source policies require trainer.candidate_log_top_k >= "
                          f"trainer.group_size for full candidate coverage (candidate_log_top_k="
                          f"{trainer.candidate_log_top_k}, group_size={trainer.group_size})")


# ------------------------------------------------------------------ candidate aggregation
@dataclass
class _StepHealth:
    total: int = 0
    correctness_supported: int = 0
    correct: int = 0
    prompt_groups: dict = field(default_factory=dict)      # prompt_index -> set(group_index)


@dataclass
class CandidateHealth:
    total: int = 0
    source_buckets: dict = field(default_factory=dict)
    steps: dict = field(default_factory=dict)

    @staticmethod
    def of(candidates: Sequence) -> "CandidateHealth":
        h = CandidateHealth()
        for rec in candidates:
            h.total += 1
            b = candidate_source_bucket(rec)
            h.source_buckets[b] = h.source_buckets.get(b, 0) + 1
            st = h.steps.setdefault(int(rec.step), _StepHealth())
            st.total += 1
            st.prompt_groups.setdefault(int(rec.prompt_index), set()).add(int(rec.group_index))
            c = candidate_correctness(rec)
            if c is not None:
                st.correctness_supported += 1
                st.correct += int(c)
        return h


def candidate_correctness(rec) -> Optional[bool]:
    """What the verifier said about one candidate, if it said anything: ``reward_metadata.correct``,
    or for the TriMul task an unextracted submission / a reward diagnostic counts as incorrect."""
    md = rec.reward_metadata
    if not isinstance(md, dict):
        return None
    if isinstance(md.get("correct"), bool):
        return md["correct"]
    if md.get("task") == "trimul" and (md.get("submission_extracted") is False or rec.reward_diagnostic is not None):
        return False
    return None


def candidate_source_bucket(rec) -> str:
    md = rec.reward_metadata
    src = md.get("source_sha256") if isinstance(md, dict) else None
    return src if isinstance(src, str) and src.strip() else UNKNOWN_SOURCE


def _fmt_steps(steps: Sequence[int]) -> str:
    head = ", ".join(str(s) for s in steps[:8])
    return head + (f", ... ({len(steps)} steps)" if len(steps) > 8 else "")


def _coverage_problem(h: CandidateHealth, steps: Sequence[int], group_size: int, groups_per_step: int,
                      scope: str) -> Optional[str]:
    missing = [s for s in steps if s not in h.steps or h.steps[s].total == 0]
    if missing:
        return f"candidate ledger missing rows for {scope} {_fmt_steps(missing)}"
    want = set(range(group_size))
    partial = [s for s in steps if len(h.steps[s].prompt_groups) != groups_per_step
               or any(g != want for g in h.steps[s].prompt_groups.values())]
    if partial:
        return f"candidate ledger lacks full group coverage for {scope} {_fmt_steps(partial)}"
    return None


# ------------------------------------------------------------------ evaluation
def evaluate_run_health(rows: Sequence, rules: dict, candidates: Optional[Sequence] = None, *,
                        group_size: Optional[int] = None, prompt_groups_per_step: Optional[int] = None) -> HealthReport:
    """Apply ``rules`` to the metrics rows (and, for the candidate-based rules, the candidate log).
    ``candidates=None`` means the log is unavailable; ``group_size`` / ``prompt_groups_per_step``
    enable the full-coverage check of the candidate-based rules."""
    rep = HealthReport()
    rules = rules or {}
    if not rows:
        rep.push("no_metrics", "fail", "no metrics rows were recorded")
    for r in rows:
        bad = [k for k in ("reward_mean", "loss", "kl", "grad_norm") if not math.isfinite(getattr(r, k, 0.0))]
        if bad:
            rep.push("non_finite", "fail", f"step {r.step} recorded non-finite {', '.join(bad)}")
            break
    rule = rules.get("reward_collapse")
    if rule:
        w = int(rule["window"])
        if len(rows) < w:
            rep.push("reward_collapse", rule["action"], f"only {len(rows)} metric rows available for {w}-step reward window")
        else:
            mean = sum(float(r.reward_mean) for r in rows[-w:]) / w
            if mean < float(rule["min"]):
                rep.push("reward_collapse", rule["action"],
                         f"trailing {w}-step mean reward {mean:.6f} fell below min {float(rule['min']):.6f}")
    rule = rules.get("dropped_rows")
    if rule:
        tot = sum(int(r.dropped_rows) for r in rows)
        if tot > int(rule["max"]):
            rep.push("dropped_rows", rule["action"], f"dropped rows {tot} exceeded max {rule['max']}")
    rule = rules.get("grad_spike")
    if rule and rows:
        pos = sorted(float(r.grad_norm) for r in rows if math.isfinite(r.grad_norm) and r.grad_norm > 0)
        if pos:
            med = pos[len(pos) // 2]
            worst = max(rows, key=lambda r: r.grad_norm if math.isfinite(r.grad_norm) else -1.0)
            factor = float(worst.grad_norm) / med
            if factor > float(rule["factor"]):
                rep.push("grad_spike", rule["action"],
                         f"grad_norm {worst.grad_norm:.6f} at step {worst.step} was {factor:.2f}x median {med:.6f}, "
                         f"above factor {float(rule['factor']):.2f}")
    action = rules.get("telemetry_dark")
    if action and rows and all(int(r.rollout_capture_tokens) == 0 for r in rows):
        rep.push("telemetry_dark", action, "off-policy drift telemetry was dark for every step")
    need = rules.get("correctness_collapse") or rules.get("source_dominance")
    health = CandidateHealth.of(candidates) if (need and candidates is not None) else None
    rule = rules.get("correctness_collapse")
    if rule:
        _correctness(rep, rows, rule, health, group_size, prompt_groups_per_step)
    rule = rules.get("source_dominance")
    if rule:
        _dominance(rep, rows, rule, health, group_size, prompt_groups_per_step)
    return rep


def _correctness(rep, rows, rule, h, group_size, groups_per_step) -> None:
    w, act = int(rule["window"]), rule["action"]
    if len(rows) < w:
        return rep.push("correctness_collapse", act, f"only {len(rows)} metric rows available for {w}-step correctness window")
    if h is None:
        return rep.push("correctness_collapse", act, "candidate ledger unavailable; cannot evaluate correctness policy")
    if h.total == 0:
        return rep.push("correctness_collapse", act, "candidate ledger is empty; cannot evaluate correctness policy")
    steps = [int(r.step) for r in rows[-w:]]
    if group_size is not None and groups_per_step is not None:
        prob = _coverage_problem(h, steps, group_size, groups_per_step, "trailing metric steps")
    else:
        missing = [s for s in steps if s not in h.steps]
        prob = f"candidate ledger missing rows for trailing metric steps {_fmt_steps(missing)}" if missing else None
    if prob:
        return rep.push("correctness_collapse", act, prob)
    unsupported = [s for s in steps if h.steps[s].correctness_supported != h.steps[s].total]
    supported = sum(h.steps[s].correctness_supported for s in steps)
    if supported == 0:
        return rep.push("correctness_collapse", act, f"no candidate correctness metadata in trailing {w} steps")
    if unsupported:
        return rep.push("correctness_collapse", act,
                        f"candidate correctness metadata unavailable for trailing metric steps {_fmt_steps(unsupported)}")
    correct = sum(h.steps[s].correct for s in steps)
    frac = correct / supported
    if frac < float(rule["min"]):
        rep.push("correctness_collapse", act, f"trailing {w}-step candidate correctness {correct}/{supported} = {frac:.3f} "
                                              f"fell below min {float(rule['min']):.3f}")


def _dominance(rep, rows, rule, h, group_size, groups_per_step) -> None:
    act = rule["action"]
    if h is None:
        return rep.push("source_dominance", act, "candidate ledger unavailable; cannot evaluate source-dominance policy")
    if h.total == 0:
        return rep.push("source_dominance", act, "candidate ledger is empty; cannot evaluate source-dominance policy")
    if group_size is not None and groups_per_step is not None:
        prob = _coverage_problem(h, [int(r.step) for r in rows], group_size, groups_per_step, "metric steps")
        if prob:
            return rep.push("source_dominance", act, prob)
    src, count = max(sorted(h.source_buckets.items()), key=lambda kv: kv[1])
    frac = count / h.total
    if frac > float(rule["max_fraction"]):
        rep.push("source_dominance", act, f"dominant candidate source {src} covered {count}/{h.total} = {frac:.3f}, "
                                          f"above max_fraction {float(rule['max_fraction']):.3f}")
