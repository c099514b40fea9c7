"""TriMul kernel-discovery task: the policy writes a GPU kernel, the reward runs it.

Reference ``crates/ferrl/src/trimul.rs``: extraction of the final fenced code
block (optionally only after ``</think>``) ``:328-382``; case list rendered as
``key: value; ...`` lines ``:280-323``; shaped reward ``:2331-2375`` with the
profile ``format_extracted 0.02 <= runnable 0.05``, ``partial_correctness
0.75``, ``correctness 1.0``, ``speed_cap 2.0`` ``:170-256``, ``:3328-3337`` and
the speed term ``baseline_ns / geomean_ns`` ``:1879-1893``; diagnostics strings
``:2377-2413``; bounded parallel verification of a group ``:3371-3430``; the
candidate and the case spec travel as sealed in-memory files ``:697-840`` and
the evaluation runs through a verifier sandbox tier (``verifier_executor``).

The evaluation driver ships with the package (``trimul_eval/ferrl_eval.py``,
counterpart of the reference's ``trimul_eval_driver.py``): its directory is the
default ``eval_dir`` (``default_eval_dir()``) and is bound read-only into the
sandbox at ``/eval``; another bundle that speaks the same protocol can be
configured instead.  The driver's grade log is the ``key: value`` line format
parsed by ``parse_eval_log``.
"""
from __future__ import annotations

import concurrent.futures as cf
import enum
import math
import os
import shutil
from dataclasses import dataclass, field
from typing import Optional, Sequence

from ..sandbox import (Bind, ProtectedOutput, ResourceLimits, RunSpec, Sandbox, SandboxInfrastructureError, SandboxOutcome, Verdict,
                       make_scratch, sealed_memfd)
from . import RewardError, RewardOutcome

FORMAT_EXTRACTED_REWARD = 0.02
RUNNABLE_REWARD = 0.05
PARTIAL_CORRECTNESS_REWARD = 0.75
CORRECTNESS_REWARD = 1.0
SPEED_REWARD_CAP = 2.0
EVAL_DRIVER_FILE = "ferrl_eval.py"
GRADE_SOCKET = "grade.sock"
TRIMUL_CASE_SEED_MAX = (1 << 32) - 1


def default_eval_dir() -> str:
    """Directory of the packaged evaluation driver."""
    return os.path.join(os.path.dirname(os.path.abspath(__file__)), "trimul_eval")


MIN_PLAUSIBLE_NS = 1000.0      # a "benchmark" faster than a microsecond is a glitch or a forged grade


class SubmissionExtractMode(str, enum.Enum):
    FINAL_FENCE = "final_fence"
    THINKING_AFTER_THINK = "thinking_after_think"


def extract_submission(completion: str, mode: SubmissionExtractMode = SubmissionExtractMode.FINAL_FENCE) -> Optional[str]:
    """The final fenced block; nothing but whitespace may follow its closing fence."""
    answer = completion
    if SubmissionExtractMode(mode) is SubmissionExtractMode.THINKING_AFTER_THINK:
        if "</think>" not in completion:
            return None
        answer = completion.rsplit("</think>", 1)[1]
    close = answer.rfind("```")
    if close < 0 or answer[close + 3:].strip():
        return None
    before = answer[:close]
    open_ = before.rfind("```")
    if open_ < 0:
        return None
    after = before[open_ + 3:]
    nl = after.find("\n")
    if nl < 0:
        return None
    code = after[nl + 1:].rstrip()
    return code if code.strip() else None


@dataclass(frozen=True)
class TrimulCase:
    seqlen: int
    bs: int
    dim: int
    hiddendim: int
    seed: int
    nomask: bool = True
    distribution: str = "normal"

    def render(self) -> str:
        return (f"seqlen: {self.seqlen}; bs: {self.bs}; dim: {self.dim}; hiddendim: {self.hiddendim}; "
                f"seed: {self.seed}; nomask: {int(self.nomask)}; distribution: {self.distribution}")


def render_spec(cases: Sequence[TrimulCase]) -> str:
    return "\n".join(c.render() for c in cases)


@dataclass
class TrimulRewardProfile:
    scheme: str = "trimul_shaped_v1"
    format_extracted: float = FORMAT_EXTRACTED_REWARD
    runnable: float = RUNNABLE_REWARD
    partial_correctness: float = PARTIAL_CORRECTNESS_REWARD
    correctness: float = CORRECTNESS_REWARD
    speed_cap: float = SPEED_REWARD_CAP
    implausible_benchmark: str = "zero"

    def validate(self) -> None:
        if self.scheme != "trimul_shaped_v1" or self.implausible_benchmark != "zero":
            raise ValueError("unknown TriMul reward scheme / implausible-benchmark policy")
        for n in ("format_extracted", "runnable", "partial_correctness", "correctness", "speed_cap"):
            v = getattr(self, n)
            if not math.isfinite(v) or v < 0:
                raise ValueError(f"trimul.reward.{n} must be finite and >= 0")
        if self.format_extracted > self.runnable:
            raise ValueError("trimul.reward.format_extracted must be <= trimul.reward.runnable")
        if self.runnable + self.partial_correctness > self.correctness:
            raise ValueError("trimul.reward.runnable + trimul.reward.partial_correctness must be <= "
                             "trimul.reward.correctness")


@dataclass
class TrimulEval:
    sandbox_ok: bool
    sandbox_verdict: str
    test_exit: Optional[int] = None
    benchmark_exit: Optional[int] = None
    tests_total: int = 0
    tests_passed: int = 0
    correct: bool = False
    has_benchmark_section: bool = False
    benchmark_means_ns: list = field(default_factory=list)
    shape_failure: bool = False

    @property
    def geomean_ns(self) -> Optional[float]:
        m = [x for x in self.benchmark_means_ns if x > 0]
        if not m or len(m) != len(self.benchmark_means_ns):
            return None
        return math.exp(sum(math.log(x) for x in m) / len(m))

    def test_fraction(self) -> float:
        return self.tests_passed / self.tests_total if self.tests_total > 0 else 0.0

    def implausible(self) -> bool:
        return any(0 <= x < MIN_PLAUSIBLE_NS for x in self.benchmark_means_ns)


def run_status_label(out: SandboxOutcome) -> str:
    """How the sandboxed run ended, as it appears in reward diagnostics (``trimul:sandbox_<label>``; the labels of
    crates/ferrl/src/trimul.rs:3293-3300)."""
    if out.verdict is Verdict.TIMEOUT:
        return "timed_out"
    if out.verdict is Verdict.SIGNALED:
        return f"signaled_{out.exit_code - 128 if out.exit_code > 128 else out.exit_code}"
    if out.verdict is Verdict.EXITED:
        return f"exited_{out.exit_code}"
    return out.verdict.value          # scratch_exceeded, launch_failed


def parse_eval_log(text: str, outcome_ok: bool = True, verdict: str = "exited") -> TrimulEval:
    """Parse the driver's ``key: value`` log. Sections: ``test-count``, ``test.<i>.status``,
    ``check: pass|fail``, ``test-exit``, ``benchmark-count``, ``benchmark.<i>.mean`` (ns),
    ``benchmark-exit``.  Unknown lines are ignored; a later duplicate key wins."""
    kv = {}
    for line in text.splitlines():
        if ":" in line:
            k, v = line.split(":", 1)
            kv[k.strip()] = v.strip()
    ev = TrimulEval(outcome_ok, verdict)

    def geti(k):
        try:
            return int(kv[k])
        except (KeyError, ValueError):
            return None
    ev.test_exit, ev.benchmark_exit = geti("test-exit"), geti("benchmark-exit")
    ev.tests_total = geti("test-count") or 0
    ev.tests_passed = sum(1 for i in range(ev.tests_total) if kv.get(f"test.{i}.status") == "pass")
    ev.shape_failure = any("shape" in kv.get(f"test.{i}.error", "").lower() for i in range(ev.tests_total))
    ev.correct = kv.get("check") == "pass" and ev.tests_total > 0 and ev.tests_passed == ev.tests_total
    n = geti("benchmark-count")
    ev.has_benchmark_section = n is not None
    for i in range(n or 0):
        try:
            ev.benchmark_means_ns.append(float(kv[f"benchmark.{i}.mean"]))
        except (KeyError, ValueError):
            ev.benchmark_means_ns.append(-1.0)
    return ev


class TrimulReward:
    """``RewardFn`` for the TriMul task. Build with ``TrimulReward(sandbox, image, eval_dir, cases)``."""

    def __init__(self, sandbox: Sandbox, image: str, eval_dir: str, cases: Sequence[TrimulCase], *,
                 benchmark_cases: Optional[Sequence[TrimulCase]] = None, scratch_root: Optional[str] = None,
                 profile: Optional[TrimulRewardProfile] = None, baseline_ns: Optional[float] = None,
                 extract_mode: SubmissionExtractMode = SubmissionExtractMode.FINAL_FENCE, wall_secs: float = 300.0,
                 scratch_max_bytes: int = 2 << 30, parallelism: int = 1, gpu: bool = True,
                 driver: Sequence[str] = ("python", "-I", "/eval/ferrl_eval.py")):
        self.sandbox, self.image, self.eval_dir = sandbox, image, eval_dir
        self.cases = list(cases)
        self.benchmark_cases = list(benchmark_cases) if benchmark_cases is not None else list(cases)
        if not self.cases:
            raise RewardError("TriMul needs at least one test case")
        self.profile = profile or TrimulRewardProfile()
        self.profile.validate()
        self.baseline_ns, self.extract_mode = baseline_ns, SubmissionExtractMode(extract_mode)
        self.scratch_root, self.wall_secs, self.scratch_max = scratch_root, wall_secs, scratch_max_bytes
        self.parallelism, self.gpu, self.driver = max(1, parallelism), gpu, list(driver)

    def with_secret_seed(self, seed: int) -> "TrimulReward":
        """Re-key every hidden case: case ``i`` gets ``seed + i`` (mod 2^32), so external scoring and
        audits never replay the inputs a policy was trained against."""
        import dataclasses
        if not 0 <= int(seed) <= TRIMUL_CASE_SEED_MAX:
            raise RewardError(f"secret seed must be between 0 and {TRIMUL_CASE_SEED_MAX}")
        self.cases = [dataclasses.replace(c, seed=(int(seed) + i) & TRIMUL_CASE_SEED_MAX) for i, c in enumerate(self.cases)]
        self.benchmark_cases = [dataclasses.replace(c, seed=(int(seed) + 7919 + i) & TRIMUL_CASE_SEED_MAX)
                                for i, c in enumerate(self.benchmark_cases)]
        return self

    def with_baseline_ns(self, ns: float) -> "TrimulReward":
        self.baseline_ns = float(ns)
        return self

    # ------------------------------------------------------------------ run
    def run_spec(self, scratch: str, fds: dict) -> RunSpec:
        binds = [Bind(self.eval_dir, "/eval", True), Bind(scratch, "/scratch", False)]
        for name, fd in fds.items():
            binds.append(Bind(f"/proc/{os.getpid()}/fd/{fd}", f"/sealed/{name}", True))
        env = [("FERRL_SUBMISSION", "/sealed/submission.py"), ("FERRL_TEST_SPEC", "/sealed/tests.txt"),
               ("FERRL_BENCH_SPEC", "/sealed/benchmarks.txt"), ("FERRL_SCRATCH", "/scratch")]
        return RunSpec(self.image, list(self.driver), binds=binds, workdir="/scratch", env=env, gpu=self.gpu,
                       limits=ResourceLimits(wall_secs=self.wall_secs), scratch_dir=scratch,
                       scratch_max_bytes=self.scratch_max,
                       protected_output=ProtectedOutput(os.path.join(scratch, GRADE_SOCKET), "/scratch/" + GRADE_SOCKET))

    def run_eval(self, submission: str) -> TrimulEval:
        scratch = make_scratch(self.scratch_root)
        fds = {}
        try:
            fds = {"submission.py": sealed_memfd("submission", submission.encode()),
                   "tests.txt": sealed_memfd("tests", render_spec(self.cases).encode()),
                   "benchmarks.txt": sealed_memfd("benchmarks", render_spec(self.benchmark_cases).encode())}
            out: SandboxOutcome = self.sandbox.run(self.run_spec(scratch, fds))
        except OSError as e:
            raise RewardError(f"TriMul eval could not be staged: {e}") from e
        except SandboxInfrastructureError as e:
            # the verifier never started: this says nothing about the candidate and must not score it
            raise RewardError(f"TriMul verifier infrastructure failed: {e}") from e
        finally:
            for fd in fds.values():
                os.close(fd)
            shutil.rmtree(scratch, ignore_errors=True)
        ok = out.verdict is Verdict.EXITED
        # the grade is what arrived on the protected socket; standard output is only the fallback of
        # sandboxes that do not offer the channel (scripted doubles)
        log = out.protected_output if out.protected_output is not None else out.stdout
        return parse_eval_log(log.decode(errors="replace"), ok, run_status_label(out))

    # --------------------------------------------------------------- reward
    def speed_value(self, geomean_ns: Optional[float]) -> float:
        if geomean_ns is None or geomean_ns <= 0:
            return 0.0
        return (self.baseline_ns / geomean_ns) if self.baseline_ns else 1e9 / geomean_ns

    def reward_from_eval(self, ev: TrimulEval) -> float:
        p = self.profile
        if not ev.sandbox_ok or ev.test_exit is None or ev.implausible():
            return 0.0
        progress = p.runnable + p.partial_correctness * ev.test_fraction()
        if ev.test_exit != 0:
            return progress
        if ev.correct and ev.has_benchmark_section and ev.benchmark_exit is not None:
            if ev.benchmark_exit == 0:
                return p.correctness + min(max(self.speed_value(ev.geomean_ns), 0.0), p.speed_cap)
            return p.correctness
        return progress

    def reward_from_extracted_eval(self, ev: TrimulEval) -> float:
        if ev.implausible():
            return 0.0
        return max(self.reward_from_eval(ev), self.profile.format_extracted)

    def diagnostic(self, ev: TrimulEval) -> Optional[str]:
        if not ev.sandbox_ok:
            return f"trimul:sandbox_{ev.sandbox_verdict}"
        if ev.test_exit is None:
            return "trimul:missing_test_exit"
        if ev.test_exit != 0:
            return "trimul:test_shape_mismatch" if ev.shape_failure else "trimul:test_process_failed"
        if ev.benchmark_exit not in (None, 0):
            return "trimul:benchmark_process_failed"
        if ev.correct and ev.geomean_ns is not None:
            return None if ev.benchmark_exit == 0 else "trimul:missing_benchmark_exit"
        if not ev.correct:
            return "trimul:test_failed" if ev.tests_total else "trimul:no_pass_grade"
        if not ev.has_benchmark_section:
            return "trimul:no_benchmark_section"
        if not ev.benchmark_means_ns:
            return "trimul:no_benchmark_means"
        return "trimul:implausible_benchmark"

    def _one(self, completion: str) -> RewardOutcome:
        sub = extract_submission(completion, self.extract_mode)
        if sub is None:
            return RewardOutcome(0.0, "trimul:no_submission", None)
        ev = self.run_eval(sub)
        meta = {"tests_passed": ev.tests_passed, "tests_total": ev.tests_total, "geomean_ns": ev.geomean_ns,
                "correct": ev.correct}
        return RewardOutcome(float(self.reward_from_extracted_eval(ev)), self.diagnostic(ev), meta)

    def reward(self, sample, completion: str) -> float:
        return self._one(completion).reward

    def reward_group(self, sample, completions):
        return [o.reward for o in self.reward_group_detailed(sample, completions)]

    def reward_group_detailed(self, sample, completions):
        """Bounded-parallel verification of a group (each candidate in its own sandbox)."""
        if self.parallelism == 1 or len(completions) <= 1:
            return [self._one(c) for c in completions]
        with cf.ThreadPoolExecutor(max_workers=self.parallelism) as ex:
            return list(ex.map(self._one, completions))

    def verify_submission(self, submission: str) -> TrimulEval:
        return self.run_eval(submission)
