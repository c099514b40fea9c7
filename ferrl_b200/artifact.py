"""Artifact audit: accept a discovered kernel only if it beats the reference kernel repeatably.

Reference ``crates/ferrl/src/artifact.rs``: 11 paired blocks, a block is a
*material win* when ``reference_ns / candidate_ns > 1.02`` (strictly), accept
iff all 11 blocks produced valid timings and at least 9 are material wins
``:34-43``, ``:1618-1648``; the order inside a block alternates
(reference-first or candidate-first) starting from a bit of the audit id so
neither side always benefits from a warm device ``:1603-1616``; the audit
re-verifies correctness with a secret case seed derived from the contract
digest; the manifest is written last, so an interrupted audit never looks
accepted ``publish_trimul_artifact :1100``.
"""
from __future__ import annotations

import hashlib
import json
import math
import os
import time
from dataclasses import asdict, dataclass, field
from typing import Callable, Optional, Sequence

ARTIFACT_CONTRACT_VERSION = 4
ARTIFACT_AUDIT_BLOCKS = 11
ARTIFACT_MATERIAL_SPEEDUP = 1.02
ARTIFACT_REQUIRED_MATERIAL_WINS = 9
ARTIFACT_ACCEPTANCE_METHOD = "paired_material_wins_v1"
MANIFEST_FILE = "artifact-manifest.json"
REPORT_FILE = "artifact-report.md"
ATTEMPT_FILE = "audit-attempt.json"


class ArtifactError(RuntimeError):
    pass


@dataclass
class AuditBlock:
    index: int
    first: str                  # "reference" | "candidate": which side ran first in this block
    reference_ns: float
    candidate_ns: float

    @property
    def paired_speedup(self) -> float:
        if not (self.reference_ns > 0 and self.candidate_ns > 0):
            return float("nan")
        return self.reference_ns / self.candidate_ns


@dataclass
class AcceptanceDecision:
    method: str
    paired_blocks: int
    material_speedup: float
    threshold_comparison: str
    required_material_wins: int
    observed_material_wins: int
    accepted: bool


def audit_id(contract: dict) -> str:
    h = hashlib.sha256(b"ferrl.artifact-audit.v1\0")
    h.update(json.dumps(contract, sort_keys=True, separators=(",", ":")).encode())
    return h.hexdigest()


def audit_seed(aid: str) -> int:
    """Secret case seed for the audit's correctness re-verification (first 4 bytes, big endian)."""
    return int(aid[:8], 16)


def audit_schedule(aid: str) -> list:
    starts_with_reference = (int(aid[:2], 16) & 1) == 0
    return ["reference" if ((i % 2 == 0) == starts_with_reference) else "candidate"
            for i in range(ARTIFACT_AUDIT_BLOCKS)]


def acceptance_from_speedups(speedups: Sequence[float]) -> AcceptanceDecision:
    valid = sum(1 for s in speedups if math.isfinite(s) and s > 0)
    wins = sum(1 for s in speedups if math.isfinite(s) and s > ARTIFACT_MATERIAL_SPEEDUP)
    return AcceptanceDecision(ARTIFACT_ACCEPTANCE_METHOD, len(speedups), ARTIFACT_MATERIAL_SPEEDUP,
                              "strict_greater_than", ARTIFACT_REQUIRED_MATERIAL_WINS, wins,
                              len(speedups) == ARTIFACT_AUDIT_BLOCKS and valid == ARTIFACT_AUDIT_BLOCKS
                              and wins >= ARTIFACT_REQUIRED_MATERIAL_WINS)


@dataclass
class ArtifactManifest:
    contract_version: int
    audit_id: str
    run_id: str
    candidate_sha256: str
    candidate_reward: float
    correct_on_secret_cases: bool
    blocks: list
    decision: dict
    accepted: bool
    run_health: str
    source_inspection: str
    source_inspection_notes: str
    created_unix: int


def publish_trimul_artifact(run_root: str, out_dir: str, candidate_source: str, candidate_reward: float,
                            verify: Callable[[str, int], bool], time_pair: Callable[[str, str], tuple],
                            *, run_health: str = "ok", source_inspection: str = "not_performed",
                            source_inspection_notes: str = "") -> ArtifactManifest:
    """Audit ``candidate_source`` and publish the verdict under ``out_dir``.

    ``verify(source, seed) -> bool`` re-checks correctness on secret-seed cases;
    ``time_pair(source, first) -> (reference_ns, candidate_ns)`` times one paired block with the
    named side running first.  Both are supplied by the caller (the sandboxed TriMul verifier on a
    real audit GPU, scripted doubles in tests)."""
    if run_health == "fail":
        raise ArtifactError("the run failed its health gate; its candidates cannot be published")
    try:
        launch = json.load(open(os.path.join(run_root, "launch.json")))
    except (OSError, json.JSONDecodeError) as e:
        raise ArtifactError(f"cannot read the run's launch.json: {e}") from e
    os.makedirs(out_dir, exist_ok=True)
    if os.path.exists(os.path.join(out_dir, MANIFEST_FILE)):
        raise ArtifactError(f"{out_dir} already holds a published artifact verdict")
    csha = hashlib.sha256(candidate_source.encode()).hexdigest()
    contract = {"contract_version": ARTIFACT_CONTRACT_VERSION, "run_id": launch.get("run_id"),
                "launch_sha256": launch.get("launch_sha256"), "candidate_sha256": csha,
                "blocks": ARTIFACT_AUDIT_BLOCKS, "material_speedup": ARTIFACT_MATERIAL_SPEEDUP,
                "required_wins": ARTIFACT_REQUIRED_MATERIAL_WINS}
    aid = audit_id(contract)
    with open(os.path.join(out_dir, ATTEMPT_FILE), "w") as f:
        json.dump({"audit_id": aid, "started_unix": int(time.time()), "contract": contract}, f, sort_keys=True)
    correct = bool(verify(candidate_source, audit_seed(aid)))
    blocks = []
    if correct:
        for i, first in enumerate(audit_schedule(aid)):
            ref_ns, cand_ns = time_pair(candidate_source, first)
            blocks.append(AuditBlock(i, first, float(ref_ns), float(cand_ns)))
    decision = acceptance_from_speedups([b.paired_speedup for b in blocks])
    if source_inspection not in ("clean", "suspicious", "not_performed"):
        raise ArtifactError(f"source_inspection must be clean, suspicious or not_performed, got {source_inspection!r}")
    # an operator who found the candidate probing processes, descriptors, the environment, the
    # network or paths outside its inputs vetoes it whatever the timings say (artifact.rs:1682)
    accepted = correct and decision.accepted and source_inspection != "suspicious"
    man = ArtifactManifest(ARTIFACT_CONTRACT_VERSION, aid, str(launch.get("run_id")), csha, float(candidate_reward),
                           correct, [dict(asdict(b), paired_speedup=b.paired_speedup) for b in blocks],
                           asdict(decision), accepted, run_health, source_inspection, source_inspection_notes,
                           int(time.time()))
    with open(os.path.join(out_dir, "candidate.py"), "w") as f:
        f.write(candidate_source)
    with open(os.path.join(out_dir, REPORT_FILE), "w") as f:
        f.write(artifact_report(man))
    tmp = os.path.join(out_dir, MANIFEST_FILE + ".tmp")           # manifest last: its presence means "complete"
    with open(tmp, "w") as f:
        json.dump(asdict(man), f, indent=2, sort_keys=True)
        f.flush()
        os.fsync(f.fileno())
    os.rename(tmp, os.path.join(out_dir, MANIFEST_FILE))
    return man


def artifact_report(m: ArtifactManifest) -> str:
    verdict = "accepted_artifact" if m.accepted else "rejected_candidate"
    if m.accepted:
        reason = "accepted: at least nine of eleven same-device pairs exceed the 2% material margin"
    elif m.source_inspection == "suspicious":
        reason = "rejected: source inspection found process/file/env/network/path probing"
    elif not m.correct_on_secret_cases:
        reason = "rejected: the candidate is not correct on the audit's secret-seed cases"
    else:
        reason = "rejected: paired audit did not establish nine material wins out of eleven"
    lines = [f"# TriMul artifact audit: {verdict}", "", reason, "", f"- run: `{m.run_id}`", f"- audit id: `{m.audit_id}`",
             f"- candidate sha256: `{m.candidate_sha256}`", f"- training reward: {m.candidate_reward:.4f}",
             f"- correct on secret-seed cases: {m.correct_on_secret_cases}",
             f"- material wins: {m.decision['observed_material_wins']} of {m.decision['paired_blocks']} "
             f"(need {m.decision['required_material_wins']} at > {m.decision['material_speedup']}x)",
             f"- run health: {m.run_health}; source inspection: {m.source_inspection}", "",
             "| block | first | reference ns | candidate ns | speedup |", "|---|---|---|---|---|"]
    for b in m.blocks:
        lines.append(f"| {b['index']} | {b['first']} | {b['reference_ns']:.0f} | {b['candidate_ns']:.0f} | "
                     f"{b['paired_speedup']:.4f} |")
    return "\n".join(lines) + "\n"
