"""Run directory, metrics stream, signed candidate log, run-health summary and
the performance regression gate.

Reference: ``crates/ferrl/src/telemetry.rs`` - ``RunDir`` file names
``:254-283``; ``Metrics`` row ``:521-678`` with non-finite sanitising ``:733``;
line-atomic fsync'd appends ``:1394-1491``; ``CandidateRecord`` ``:794-835``
digested under a domain tag and Ed25519-signed against the launch digest
``:1027-1088``; anomalies (NonFinite, GradSpike > 8x median, RewardStall,
DroppedRows, TelemetryDark) ``:1526-1703``; ``RegressionBudget`` ``:1711-1763``
and ``compare_metrics`` ``:2071`` (mean step-seconds ratio <= 1.10, peak memory
<= 1.0x + 64 MiB).

B200 additions: per-phase CUDA-event timers (``PhaseTimer``) and device memory
probes using the reference's phase labels, so ``metrics.jsonl`` carries
device-timed phase durations next to the host wall clock.
"""
from __future__ import annotations

import dataclasses
import hashlib
import json
import logging
import math
import os
import statistics
import time
from dataclasses import dataclass, field
from typing import Any, Optional, Sequence

log = logging.getLogger("ferrl_b200")

GRAD_SPIKE_FACTOR = 8.0
STALL_MIN_STEPS = 5
STALL_ZERO_STD_FRAC = 0.9
STALL_TREND_EPS = 1e-4
F32_MAX = 3.4028234663852886e38


def init_tracing(level: Optional[str] = None) -> None:
    """Configure logging once; level from ``FERRL_LOG`` (default INFO)."""
    lvl = (level or os.environ.get("FERRL_LOG", "INFO")).upper()
    logging.basicConfig(level=getattr(logging, lvl, logging.INFO),
                        format="%(asctime)s %(levelname)s %(name)s %(message)s")


class run_span:
    """Context manager that tags every log record with rank/world (and step)."""

    def __init__(self, rank: int, world: int, step: Optional[int] = None):
        self.extra = f"[rank {rank}/{world}" + (f" step {step}]" if step is not None else "]")

    def __enter__(self):
        self._old = logging.getLogRecordFactory()
        extra, old = self.extra, self._old

        def factory(*a, **k):
            rec = old(*a, **k)
            rec.msg = f"{extra} {rec.msg}"
            return rec
        logging.setLogRecordFactory(factory)
        return self

    def __exit__(self, *exc):
        logging.setLogRecordFactory(self._old)
        return False


def nan_to_num(x: float) -> float:
    """JSON-safe float: NaN -> 0, +/-inf -> +/-f32::MAX."""
    if x != x:
        return 0.0
    if x == math.inf:
        return F32_MAX
    if x == -math.inf:
        return -F32_MAX
    return float(x)


@dataclass
class Metrics:
    step: int = 0
    loss: float = 0.0
    reward_mean: float = 0.0
    reward_std: float = 0.0
    frac_reward_zero_std: float = 0.0
    kl: float = 0.0
    clip_ratio: float = 0.0
    clip_ratio_low: float = 0.0
    clip_ratio_high: float = 0.0
    frac_truncated: float = 0.0
    completion_len: float = 0.0
    completion_len_max: float = 0.0
    rollout_ratio_mean: float = 0.0
    rollout_logratio_mean: float = 0.0
    rollout_ratio_max: float = 0.0
    frac_rollout_ratio_capped: float = 0.0
    rollout_capture_tokens: int = 0
    dropped_rows: int = 0
    live_groups: int = 0
    skipped_groups: int = 0
    grad_norm: float = 0.0
    lr: float = 0.0
    beta: float = 0.0
    step_secs: float = 0.0
    tokens_per_sec: float = 0.0
    rank: int = 0
    world_size: int = 1
    cuda_mem_start_used_bytes: int = 0
    cuda_mem_peak_used_bytes: int = 0
    cuda_mem_end_used_bytes: int = 0
    cuda_mem_total_bytes: int = 0
    cuda_mem_peak_delta_bytes: int = 0      # peak increase over the step's first probe; 0 = unmeasured or no increase
    cuda_mem_probe_events: list = field(default_factory=list)
    decoder_cache_bytes: int = 0
    phase_ms: dict = field(default_factory=dict)
    nonfinite_fields: list = field(default_factory=list)

    def sanitized(self) -> dict:
        d = dataclasses.asdict(self)
        bad = []
        for k, v in list(d.items()):
            if isinstance(v, float) and not math.isfinite(v):
                bad.append(k)
                d[k] = nan_to_num(v)
        d["nonfinite_fields"] = sorted(set(self.nonfinite_fields) | set(bad))
        return d

    @staticmethod
    def from_json(d: dict) -> "Metrics":
        names = {f.name for f in dataclasses.fields(Metrics)}
        return Metrics(**{k: v for k, v in d.items() if k in names})


def _append_line(path: str, line: str) -> None:
    data = (line + "\n").encode()
    fd = os.open(path, os.O_WRONLY | os.O_APPEND | os.O_CREAT, 0o644)
    try:
        os.write(fd, data)  # one write call => line-atomic with O_APPEND
        os.fsync(fd)
    finally:
        os.close(fd)


class MetricsWriter:
    def __init__(self, path: str):
        self.path = path

    def append(self, m: Metrics) -> None:
        _append_line(self.path, json.dumps(m.sanitized(), sort_keys=True, allow_nan=False))


def read_metrics(path: str) -> list[Metrics]:
    out = []
    with open(path, encoding="utf-8") as f:
        for i, line in enumerate(f):
            if not line.strip():
                continue
            try:
                out.append(Metrics.from_json(json.loads(line)))
            except (json.JSONDecodeError, TypeError) as e:
                raise ValueError(f"{path}:{i + 1}: malformed metrics row: {e}") from e
    return out


class RunDir:
    METRICS_FILE = "metrics.jsonl"
    CANDIDATES_FILE = "candidates.jsonl"
    LAUNCH_FILE = "launch.json"
    PROMPT_FILE = "prompt.txt"
    PROMPT_SHA256_FILE = "prompt.sha256"
    CONFIG_FILE = "config.json"
    EVAL_REPORT_FILE = "eval-report.json"
    CHECKPOINTS_DIR = "checkpoints"

    def __init__(self, root: str, run_id: str):
        self.root = root
        self.run_id = run_id

    @staticmethod
    def create(out_dir: str, run_id: str) -> "RunDir":
        root = os.path.join(out_dir, run_id)
        try:
            os.makedirs(root, exist_ok=False)
        except FileExistsError:
            raise FileExistsError(f"run directory {root} already exists; refusing to overwrite a run") from None
        os.makedirs(os.path.join(root, RunDir.CHECKPOINTS_DIR))
        return RunDir(root, run_id)

    @staticmethod
    def open(root: str, run_id: Optional[str] = None) -> "RunDir":
        """Continue an existing run: ``open(run_root)`` or, as the reference spells it, ``open(out_dir, run_id)``.
        A missing directory is an error (a mistyped run id must not start an empty "resume"); the eager layout
        (the checkpoints directory) is materialised as ``create`` does (telemetry.rs:2927-2936, :3245-3264)."""
        if run_id is not None:
            root = os.path.join(root, run_id)
        if not os.path.isdir(root):
            raise FileNotFoundError(f"run directory {root} does not exist")
        rd = RunDir(root, os.path.basename(os.path.normpath(root)))
        os.makedirs(rd.checkpoints_dir, exist_ok=True)
        return rd

    def path(self, name: str) -> str:
        return os.path.join(self.root, name)

    @property
    def metrics_path(self):
        return self.path(self.METRICS_FILE)

    @property
    def candidates_path(self):
        return self.path(self.CANDIDATES_FILE)

    @property
    def checkpoints_dir(self):
        return self.path(self.CHECKPOINTS_DIR)

    def write_json_once(self, name: str, obj: Any) -> str:
        """Immutable JSON file (launch.json, config.json): written via temp +
        rename, never replaced."""
        p = self.path(name)
        if os.path.exists(p):
            raise FileExistsError(f"{p} already exists and is immutable")
        tmp = p + ".tmp"
        with open(tmp, "w", encoding="utf-8") as f:
            json.dump(obj, f, sort_keys=True, indent=2)
            f.flush()
            os.fsync(f.fileno())
        os.rename(tmp, p)
        return p

    def write_prompt(self, text: str) -> str:
        sha = hashlib.sha256(text.encode()).hexdigest()
        with open(self.path(self.PROMPT_FILE), "w", encoding="utf-8") as f:
            f.write(text)
        with open(self.path(self.PROMPT_SHA256_FILE), "w") as f:
            f.write(sha + "\n")
        return sha


# ------------------------------------------------------------- candidates
CANDIDATE_DIGEST_DOMAIN = b"ferrl.candidate-record.v1"


@dataclass
class CandidateRecord:
    step: int
    rank: int
    world_size: int
    prompt_index: int
    group_index: int
    reward: float
    completion_len_tokens: int
    completion: str
    reward_diagnostic: Optional[str] = None
    reward_metadata: Optional[Any] = None
    launch_sha256: Optional[str] = None
    record_sha256: Optional[str] = None
    record_signature: Optional[str] = None

    def body(self) -> dict:
        d = {k: v for k, v in dataclasses.asdict(self).items()
             if k not in ("record_sha256", "record_signature") and v is not None}
        return d

    def digest(self) -> str:
        h = hashlib.sha256()
        h.update(CANDIDATE_DIGEST_DOMAIN + b"\0")
        h.update(json.dumps(self.body(), sort_keys=True, separators=(",", ":")).encode())
        return h.hexdigest()


class CandidateSigner:
    """Ed25519 signer bound to one launch digest. The public key is published in
    ``launch.json``; a record is authentic when its digest matches its body and
    the signature verifies under that key."""

    def __init__(self, launch_sha256: str, seed: Optional[bytes] = None):
        from nacl.signing import SigningKey
        self._key = SigningKey(seed) if seed is not None else SigningKey.generate()
        self.launch_sha256 = launch_sha256

    @property
    def public_key_hex(self) -> str:
        return self._key.verify_key.encode().hex()

    def sign(self, rec: CandidateRecord) -> CandidateRecord:
        rec.launch_sha256 = self.launch_sha256
        rec.record_sha256 = rec.digest()
        rec.record_signature = self._key.sign(bytes.fromhex(rec.record_sha256)).signature.hex()
        return rec


def verify_candidate(rec: CandidateRecord, public_key_hex: str, launch_sha256: str) -> None:
    from nacl.exceptions import BadSignatureError
    from nacl.signing import VerifyKey
    if rec.launch_sha256 != launch_sha256:
        raise ValueError("candidate is bound to a different launch")
    if rec.record_sha256 is None or rec.record_signature is None:
        raise ValueError("candidate is unsigned")
    if rec.digest() != rec.record_sha256:
        raise ValueError("candidate digest does not match its body")
    try:
        VerifyKey(bytes.fromhex(public_key_hex)).verify(bytes.fromhex(rec.record_sha256),
                                                        bytes.fromhex(rec.record_signature))
    except (BadSignatureError, ValueError) as e:
        raise ValueError(f"candidate signature is invalid: {e}") from e


class CandidateWriter:
    """Appends candidate rows.  With a signer every row is bound to the launch; such a writer refuses a ledger that
    already holds rows, because the process-local key that signed them is gone and mixed provenance could not be
    told apart (telemetry.rs:1229-1250).  A non-finite reward is refused before anything is written
    (telemetry.rs:3152-3185): the ledger is strict JSON."""

    def __init__(self, path: str, signer: Optional[CandidateSigner] = None):
        self.path = path
        self.signer = signer
        if signer is not None and os.path.exists(path) and os.path.getsize(path) != 0:
            raise ValueError(f"refuse to bind launch-authenticated candidate appends to non-empty ledger {path}; "
                             "the original process-local signing capability is unavailable")

    def append(self, rec: CandidateRecord) -> None:
        if not math.isfinite(float(rec.reward)):
            raise ValueError(f"candidate reward {rec.reward!r} is not finite")
        if self.signer is not None:
            rec = self.signer.sign(rec)
        d = {k: v for k, v in dataclasses.asdict(rec).items() if v is not None}
        _append_line(self.path, json.dumps(d, sort_keys=True, allow_nan=False))

    def mark(self) -> int:
        """Current end of the ledger: what ``rollback`` cuts back to."""
        try:
            return os.path.getsize(self.path)
        except OSError:
            return 0

    def rollback(self, mark: int) -> None:
        """Drop every row appended since ``mark`` (a failed window must leave no candidate rows behind:
        its completions belong to a policy state that was rolled back; reference trainer.rs:7819)."""
        if not os.path.exists(self.path) or os.path.getsize(self.path) <= mark:
            return
        with open(self.path, "r+b") as f:
            f.truncate(mark)
            f.flush()
            os.fsync(f.fileno())


def read_candidates(path: str) -> list[CandidateRecord]:
    out = []
    if not os.path.exists(path):
        return out
    with open(path, encoding="utf-8") as f:
        for line in f:
            if line.strip():
                out.append(CandidateRecord(**json.loads(line)))
    return out


# ------------------------------------------------------------------ health
@dataclass
class Anomaly:
    kind: str  # non_finite | grad_spike | reward_stall | dropped_rows | telemetry_dark
    detail: dict = field(default_factory=dict)

    def __str__(self):
        d = self.detail
        if self.kind == "non_finite":
            return f"non-finite `{d['field']}` saturated at step {d['step']}"
        if self.kind == "grad_spike":
            return (f"grad_norm spike {d['grad_norm']:.3f} at step {d['step']} "
                    f"({d['grad_norm'] / d['median']:.1f}x median {d['median']:.3f})")
        if self.kind == "reward_stall":
            return (f"reward stalled: {100 * d['mean_frac_zero_std']:.0f}% groups zero-std, "
                    f"trend {d['reward_trend']:+.4f}")
        if self.kind == "dropped_rows":
            return f"{d['total']} completion rows were dropped (fully masked)"
        return "telemetry dark: no metrics rows were recorded"


@dataclass
class RunSummary:
    steps: int
    reward_first: float
    reward_last: float
    reward_best: float
    mean_step_secs: float
    mean_tokens_per_sec: float
    final_grad_norm: float
    peak_mem_bytes: int
    anomalies: list

    def healthy(self) -> bool:
        return not self.anomalies


def detect_anomalies(rows: Sequence[Metrics]) -> list[Anomaly]:
    out: list[Anomaly] = []
    if not rows:
        return [Anomaly("telemetry_dark")]
    for r in rows:
        for f in r.nonfinite_fields:
            out.append(Anomaly("non_finite", {"step": r.step, "field": f}))
    norms = [r.grad_norm for r in rows if r.grad_norm > 0]
    if len(norms) >= 3:
        med = statistics.median(norms)
        if med > 0:
            for r in rows:
                if r.grad_norm > GRAD_SPIKE_FACTOR * med:
                    out.append(Anomaly("grad_spike", {"step": r.step, "grad_norm": r.grad_norm, "median": med}))
    if len(rows) >= STALL_MIN_STEPS:
        mz = sum(r.frac_reward_zero_std for r in rows) / len(rows)
        n = len(rows)
        xs = list(range(n))
        mx, my = (n - 1) / 2, sum(r.reward_mean for r in rows) / n
        den = sum((x - mx) ** 2 for x in xs)
        trend = sum((x - mx) * (r.reward_mean - my) for x, r in zip(xs, rows)) / den if den else 0.0
        if mz >= STALL_ZERO_STD_FRAC and abs(trend) <= STALL_TREND_EPS:
            out.append(Anomaly("reward_stall", {"mean_frac_zero_std": mz, "reward_trend": trend}))
    dropped = sum(r.dropped_rows for r in rows)
    if dropped > 0:
        out.append(Anomaly("dropped_rows", {"total": dropped}))
    return out


def summarize(rows: Sequence[Metrics]) -> RunSummary:
    an = detect_anomalies(rows)
    if not rows:
        return RunSummary(0, 0, 0, 0, 0, 0, 0, 0, an)
    return RunSummary(
        steps=len(rows), reward_first=rows[0].reward_mean, reward_last=rows[-1].reward_mean,
        reward_best=max(r.reward_mean for r in rows),
        mean_step_secs=sum(r.step_secs for r in rows) / len(rows),
        mean_tokens_per_sec=sum(r.tokens_per_sec for r in rows) / len(rows),
        final_grad_norm=rows[-1].grad_norm,
        peak_mem_bytes=max(r.cuda_mem_peak_used_bytes for r in rows), anomalies=an)


# ------------------------------------------------------------ perf gate
@dataclass
class RegressionBudget:
    require_live_update: bool = True
    require_timing: bool = True
    require_cuda_memory: bool = True
    allow_health_warnings: bool = False
    warmup_steps: int = 0
    min_positive_grad_steps: int = 1
    max_mean_step_secs_ratio: float = 1.10
    max_mean_step_secs_abs_slack: float = 0.0
    max_cuda_peak_used_ratio: float = 1.0
    max_cuda_peak_used_abs_slack_bytes: int = 64 * 1024 * 1024
    max_final_grad_norm_rel_drift: Optional[float] = None


@dataclass
class RegressionReport:
    passed: bool
    failures: list
    baseline_mean_step_secs: float
    candidate_mean_step_secs: float
    baseline_peak_bytes: int
    candidate_peak_bytes: int


def compare_metrics(baseline: Sequence[Metrics], candidate: Sequence[Metrics],
                    budget: Optional[RegressionBudget] = None) -> RegressionReport:
    b = budget or RegressionBudget()
    fails = []
    if not baseline:
        fails.append("baseline metrics stream is empty")
    if not candidate:
        fails.append("candidate metrics stream is empty")
    if fails:
        return RegressionReport(False, fails, 0, 0, 0, 0)
    bs, cs = baseline[b.warmup_steps:], candidate[b.warmup_steps:]
    if not bs or not cs:
        return RegressionReport(False, ["no rows left after warmup_steps"], 0, 0, 0, 0)
    if b.require_live_update:
        for name, rows in (("baseline", bs), ("candidate", cs)):
            if sum(1 for r in rows if r.grad_norm > 0) < b.min_positive_grad_steps:
                fails.append(f"{name} has fewer than {b.min_positive_grad_steps} steps with a live update")
    bm = sum(r.step_secs for r in bs) / len(bs)
    cm = sum(r.step_secs for r in cs) / len(cs)
    if b.require_timing:
        if bm <= 0 or cm <= 0:
            fails.append("step timing is missing (step_secs <= 0)")
        elif cm > bm * b.max_mean_step_secs_ratio + b.max_mean_step_secs_abs_slack:
            fails.append(f"mean step seconds {cm:.4f} exceeds budget {b.max_mean_step_secs_ratio:.2f}x of {bm:.4f}")
    bp = max(r.cuda_mem_peak_used_bytes for r in bs)
    cp = max(r.cuda_mem_peak_used_bytes for r in cs)
    if b.require_cuda_memory:
        if bp == 0 or cp == 0:
            fails.append("CUDA memory telemetry is missing (enable gpu_memory_probe)")
        elif cp > bp * b.max_cuda_peak_used_ratio + b.max_cuda_peak_used_abs_slack_bytes:
            fails.append(f"peak memory {cp} exceeds budget of {bp} x{b.max_cuda_peak_used_ratio} + "
                         f"{b.max_cuda_peak_used_abs_slack_bytes}")
    if not b.allow_health_warnings:
        for a in detect_anomalies(cs):
            if a.kind != "dropped_rows":
                fails.append(f"candidate run health: {a}")
    if b.max_final_grad_norm_rel_drift is not None and bs[-1].grad_norm > 0:
        drift = abs(cs[-1].grad_norm - bs[-1].grad_norm) / bs[-1].grad_norm
        if drift > b.max_final_grad_norm_rel_drift:
            fails.append(f"final grad-norm drift {drift:.4f} exceeds {b.max_final_grad_norm_rel_drift}")
    return RegressionReport(not fails, fails, bm, cm, bp, cp)


def compare_distributed_metrics(baselines: Sequence[Sequence[Metrics]], candidates: Sequence[Sequence[Metrics]],
                                budget: Optional[RegressionBudget] = None) -> list[RegressionReport]:
    """Rank-by-rank comparison; rank counts must match."""
    if len(baselines) != len(candidates):
        raise ValueError("baseline and candidate runs have different rank counts")
    return [compare_metrics(b, c, budget) for b, c in zip(baselines, candidates)]


def aggregate_world_rows(stream: str, ranks: Sequence[Sequence[Metrics]], budget: RegressionBudget,
                         failures: list) -> list:
    """One row per step for a whole data-parallel job: the slowest rank's ``step_secs``, the largest
    peak memory, summed tokens and dropped rows, rank 0's update statistics.  Every rank must have
    logged the same steps; missing timing or memory telemetry on ANY rank is a failure."""
    if not ranks or not ranks[0]:
        failures.append(f"{stream} metrics stream is empty")
        return []
    n = len(ranks[0])
    for r, rows in enumerate(ranks):
        if len(rows) != n:
            failures.append(f"{stream} rank {r} logged {len(rows)} steps, rank 0 logged {n}")
    n = min(len(rows) for rows in ranks)
    if n == 0:
        failures.append(f"{stream} metrics stream is empty")
        return []
    flat = [m for rows in ranks for m in rows]
    if budget.require_timing and any(not math.isfinite(m.step_secs) or m.step_secs <= 0 for m in flat):
        failures.append(f"{stream}: step timing is missing on at least one rank")
    if budget.require_cuda_memory and any(m.cuda_mem_peak_used_bytes == 0 for m in flat):
        failures.append(f"{stream}: CUDA memory telemetry is missing on at least one rank")
    out = []
    for i in range(n):
        row = [rows[i] for rows in ranks]
        if any(m.step != row[0].step for m in row):
            failures.append(f"{stream} row {i}: ranks disagree on the step index {[m.step for m in row]}")
        agg = dataclasses.replace(row[0])
        agg.step_secs = max(m.step_secs for m in row)
        agg.cuda_mem_peak_used_bytes = max(m.cuda_mem_peak_used_bytes for m in row)
        agg.dropped_rows = sum(m.dropped_rows for m in row)
        agg.tokens_per_sec = sum(m.tokens_per_sec for m in row)
        agg.reward_mean = sum(m.reward_mean for m in row) / len(row)
        out.append(agg)
    return out


def compare_world_max_metrics(baseline_ranks: Sequence[Sequence[Metrics]], candidate_ranks: Sequence[Sequence[Metrics]],
                              budget: Optional[RegressionBudget] = None) -> RegressionReport:
    """Gate a multi-rank run as ONE job: per-rank health must not differ, then the world rows
    (``aggregate_world_rows``) are compared like a single stream."""
    b = budget or RegressionBudget()
    fails: list = []
    if len(baseline_ranks) != len(candidate_ranks):
        fails.append(f"baseline has {len(baseline_ranks)} ranks, candidate has {len(candidate_ranks)}")
    elif not b.allow_health_warnings:
        for r, (br, cr) in enumerate(zip(baseline_ranks, candidate_ranks)):
            ba, ca = [str(a) for a in detect_anomalies(br)], [str(a) for a in detect_anomalies(cr)]
            if ba != ca:
                fails.append(f"rank {r}: health findings differ ({len(ba)} in baseline, {len(ca)} in candidate)")
    base = aggregate_world_rows("baseline", baseline_ranks, b, fails)
    cand = aggregate_world_rows("candidate", candidate_ranks, b, fails)
    rep = compare_metrics(base, cand, b)
    rep.failures = fails + [f for f in rep.failures if f not in fails]
    rep.passed = not rep.failures
    return rep


# ------------------------------------------------------- device probes
def cuda_memory_snapshot(device=None) -> Optional[tuple[int, int]]:
    """``(used_bytes, total_bytes)`` from the driver, or ``None`` without a GPU."""
    import torch
    if not torch.cuda.is_available():
        return None
    free, total = torch.cuda.mem_get_info(device)
    return total - free, total


class GpuMemoryProbe:
    """Records used device bytes at named phase labels (``rollout_prefill_start``
    ... ``optimizer_end``), as the reference's probe does."""

    def __init__(self, enabled: bool, device=None):
        self.enabled = enabled and cuda_memory_snapshot(device) is not None
        self.device = device
        self.events: list = []
        self.start = self.peak = self.end = self.total = 0

    def record(self, label: str) -> None:
        if not self.enabled:
            return
        used, total = cuda_memory_snapshot(self.device)
        if not self.events:
            self.start = used
        self.peak = max(self.peak, used)
        self.end, self.total = used, total
        self.events.append({"label": label, "used_bytes": used})


class PhaseTimer:
    """CUDA-event (or host clock on CPU) timers keyed by phase label."""

    def __init__(self, device):
        import torch
        self.cuda = device is not None and getattr(device, "type", "cpu") == "cuda"
        self.torch = torch
        self.open: dict = {}
        self.pairs: list = []
        self.ms: dict = {}

    def start(self, label: str):
        if self.cuda:
            self.torch.cuda.nvtx.range_push(label)      # lets a profiler filter launches by phase
            e = self.torch.cuda.Event(enable_timing=True)
            e.record()
            self.open[label] = e
        else:
            self.open[label] = time.perf_counter()

    def stop(self, label: str):
        s = self.open.pop(label)
        if self.cuda:
            e = self.torch.cuda.Event(enable_timing=True)
            e.record()
            self.torch.cuda.nvtx.range_pop()
            self.pairs.append((label, s, e))
        else:
            self.ms[label] = self.ms.get(label, 0.0) + (time.perf_counter() - s) * 1e3

    def collect(self) -> dict:
        if self.cuda and self.pairs:
            self.torch.cuda.synchronize()
            for label, s, e in self.pairs:
                self.ms[label] = self.ms.get(label, 0.0) + s.elapsed_time(e)
            self.pairs = []
        out, self.ms = self.ms, {}
        return out
