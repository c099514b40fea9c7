"""Discovery SDK: the small stable surface for "train a policy on a verifiable task and give me
its best candidates".

Reference ``crates/ferrl/src/discovery.rs``: ``DiscoveryTask`` ``:782-831``,
``DiscoveryConfig`` + builder ``:835-1029``, ``Discovery::run`` ``:1064-1140``,
outcomes ``:1172-1380``, manifest-last publication ``:1857-2040``.  The engine
underneath is ``ferrl_b200.orchestration``; this module only fixes a narrow,
typed entry point and an outcome record.
"""
from __future__ import annotations

import json
import os
from dataclasses import dataclass, field
from typing import Optional, Sequence

from .config import PolicyCfg, RunConfig, TrainerConfig
from .orchestration import TrainOutcome, run_cli_train_setup
from .rewards import RewardFn, Sample


@dataclass
class DiscoveryTask:
    name: str
    samples: Sequence[Sample]
    reward_fn: RewardFn
    eval_samples: Sequence[Sample] = ()


@dataclass
class DiscoveryConfig:
    model_dir: str
    out_dir: str = "runs"
    device: str = "cpu"
    trainer: TrainerConfig = field(default_factory=TrainerConfig)
    policy: PolicyCfg = field(default_factory=PolicyCfg)
    candidate_top_k: int = 4
    allow_dirty: bool = True

    class Builder:
        def __init__(self, model_dir: str):
            self._c = DiscoveryConfig(model_dir)

        def out_dir(self, p):
            self._c.out_dir = p
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

        def build(self) -> "DiscoveryConfig":
            self._c.trainer.candidate_log_top_k = self._c.candidate_top_k
            self._c.trainer.validate()
            if self._c.candidate_top_k < 1:
                raise ValueError("candidate_top_k must be >= 1")
            return self._c


@dataclass
class DiscoveryOutcome:
    run_dir: str
    stop: str
    steps_run: int
    health_verdict: str
    best: list                     # CandidateRecord, best first
    eval_improvement: Optional[float]

    def to_json(self):
        return {"run_dir": self.run_dir, "stop": self.stop, "steps_run": self.steps_run,
                "health_verdict": self.health_verdict, "eval_improvement": self.eval_improvement,
                "best": [{"reward": c.reward, "step": c.step, "completion": c.completion} for c in self.best]}


class Discovery:
    def __init__(self, task: DiscoveryTask, config: DiscoveryConfig, tokenizer=None, model_and_identity=None):
        self.task, self.config, self.tokenizer, self.model_and_identity = task, config, tokenizer, model_and_identity

    def run(self) -> DiscoveryOutcome:
        import ferrl_b200.orchestration as orch
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
                                                    model_and_identity=self.model_and_identity)
        finally:
            orch.build_task = orig
        res = DiscoveryOutcome(out.run_dir, out.stop, out.steps_run, out.health.verdict,
                               out.candidates[:c.candidate_top_k],
                               None if out.eval_report is None else out.eval_report.improvement())
        tmp = os.path.join(out.run_dir, "discovery-outcome.json.tmp")       # written last
        with open(tmp, "w") as f:
            json.dump(res.to_json(), f, indent=2, sort_keys=True)
        os.rename(tmp, os.path.join(out.run_dir, "discovery-outcome.json"))
        return res
