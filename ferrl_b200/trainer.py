"""The GRPO training loop.

One optimizer step (a *window*) is: select prompts -> roll out groups -> score
rewards -> group-relative advantages and masks -> (reference log-probs for the
KL term) -> ``mu`` inner epochs of {grad-bearing scoring forward, loss,
backward, gradient reduce, coverage canary, global-norm clip, AdamW} ->
metrics row -> optional checkpoint -> preemption poll.

Reference: ``crates/ferrl/src/trainer.rs`` - ``run`` ``:7032-7217``,
``run_window`` ``:7384-7580``, ``select_prompt`` ``:7582-7626``,
``collect_group`` ``:8102-8343``, ``materialize_collected_group``
``:8347-8431``, distributed same-prompt advantages ``:8543-8615``,
``accumulate_step`` ``:8661-8819``, ``item_backward`` ``:8879-9047``,
``grpo_loss`` ``:9951-9985``, ``global_grad_norm`` ``:10032``, checkpoint write
``:7873-7981``, preemption ``:8036-8056``, rollback ``:5120-5290``.

Differences that come from designing for B200 rather than translating:

* an accumulation item holds ``prompts_per_item`` prompts that are rolled out
  and scored as ONE batch (the reference handles one group at a time);
* with ``mu == 1`` the old-policy log-probs are the detached values of the
  grad-bearing forward itself (bit-identical to a separate detached forward
  over unchanged weights), which removes one full forward per step;
* control scalars of a window travel in one packed exchange;
* on GPUs under data parallelism the reduce/clip/AdamW tail is the fused
  peer-memory kernel (``parallel.dp.FusedDpStep``) instead of per-tensor NCCL
  calls, with a deterministic rank order so ranks stay in bitwise lockstep.
"""
from __future__ import annotations

import enum
import math
import threading
import time
from dataclasses import dataclass, field
from typing import Callable, Optional, Protocol, Sequence

import torch

from . import grpo
from .checkpoint import (CheckpointBinding, CheckpointError, CheckpointMismatch, LoadedCheckpoint,
                         latest_checkpoint, prepare_checkpoint, save_checkpoint)
from .comm import Comm, CommError, PeerFailure, SoloComm
from .config import RewardGroupScope, TrainerConfig
from .grpo import ImportanceSamplingLevel, LossConfig, LossType, ScaleRewards
from .optim import AdamWParams, FerrlAdamW, OptimizerState
from .policy import GenConfig, Policy, Rollout, validate_generated_rollout_semantics
from .rewards import RewardError, RewardFn, Sample
from .telemetry import (CandidateRecord, CandidateWriter, GpuMemoryProbe, Metrics, MetricsWriter, PhaseTimer,
                        RunDir, log)


class TokenizerLike(Protocol):
    def encode(self, text: str) -> list[int]: ...
    def decode(self, ids: Sequence[int]) -> str: ...


class RunStop(enum.Enum):
    COMPLETED = "completed"
    PREEMPTED = "preempted"


# a rank whose backward raised enters the fused data-parallel step with this "uncovered" count (exact in
# float32, far above any real tensor count) so that every rank learns of it from the kernel's world-wide sum
PEER_FAILED_COUNT = float(2 ** 20)


class TrainerError(RuntimeError):
    pass


class GradCoverageError(TrainerError):
    """A trainable tensor received no gradient, or a non-finite one."""


class MustDiscard(TrainerError):
    """Rollback itself failed: live state is undefined, the trainer must be dropped."""


@dataclass
class PromptSelection:
    sample_idx: int
    prompt_index: int
    rollout_global_row_base: int


@dataclass
class CollectedGroup:
    selection: PromptSelection
    sample: Sample
    prompt_ids: list
    rollout: Rollout
    completions: list
    rewards: list
    outcomes: list
    advantages: list
    mask: torch.Tensor          # [G, N] float32 (host)
    truncated: int
    completion_tokens: int

    @property
    def live(self) -> bool:
        return any(a != 0.0 for a in self.advantages)


@dataclass
class LiveItem:
    rollouts: list              # list[Rollout], one per live group
    advantages: torch.Tensor    # [R] device
    mask: torch.Tensor          # [R, N] device
    logp_old: Optional[torch.Tensor]
    logp_ref: Optional[torch.Tensor]
    tis_w: Optional[torch.Tensor]
    rollout_lp: Optional[torch.Tensor]  # behaviour log-probs [R, N] device


@dataclass
class WindowStats:
    rewards: list = field(default_factory=list)
    group_stds: list = field(default_factory=list)
    zero_std_groups: int = 0
    groups: int = 0
    live_groups: int = 0
    truncated: int = 0
    rows: int = 0
    completion_tokens: int = 0
    completion_len_max: int = 0
    dropped_rows: int = 0
    ratio_sum: float = 0.0
    logratio_sum: float = 0.0
    ratio_max: float = 0.0
    ratio_capped: float = 0.0
    ratio_tokens: float = 0.0


def length_mask(rollout: Rollout) -> torch.Tensor:
    N = rollout.width
    lens = torch.as_tensor(rollout.completion_lens)
    return (torch.arange(N)[None, :] < lens[:, None]).to(torch.float32)


def mask_truncated_rows(rollout: Rollout, eos: Optional[int], mask: torch.Tensor) -> int:
    """Zero the mask rows of completions that fill the whole width without
    ending in EOS (reference trainer.rs:9432-9461). Inert when ``eos`` is None."""
    if eos is None:
        return 0
    N = rollout.width
    n = 0
    for i, ln in enumerate(rollout.completion_lens):
        if ln == N and int(rollout.token_ids[i, rollout.prompt_len + ln - 1]) != eos:
            mask[i].zero_()
            n += 1
    return n


def global_grad_norm(grads: Sequence[torch.Tensor]) -> float:
    """sqrt(sum g^2) accumulated in float64."""
    if not grads:
        return 0.0
    total = torch.zeros((), dtype=torch.float64, device=grads[0].device)
    for g in grads:
        total += g.double().pow(2).sum()
    return float(total.sqrt().item())


def grad_coverage(params: Sequence[torch.nn.Parameter]) -> tuple[list[int], list[int]]:
    """Indices of trainable tensors with a missing / non-finite gradient
    (reference nn.rs:342-375)."""
    missing = [i for i, p in enumerate(params) if p.grad is None]
    nonfinite = []
    present = [(i, p.grad) for i, p in enumerate(params) if p.grad is not None]
    if present:
        flags = torch.stack([torch.isfinite(g).all() for _, g in present]).cpu().tolist()
        nonfinite = [i for (i, _), ok in zip(present, flags) if not ok]
    return missing, nonfinite


class Trainer:
    def __init__(self, policy: Policy, tokenizer: TokenizerLike, reward_fn: RewardFn, samples: Sequence[Sample],
                 config: TrainerConfig, *, comm: Optional[Comm] = None, topology: str = "dp",
                 run_dir: Optional[RunDir] = None, binding: Optional[CheckpointBinding] = None,
                 candidate_writer: Optional[CandidateWriter] = None, adam_eps: float = 1e-8,
                 fused_dp_step=None, parallel_runtime=None, lockstep_model_calls: bool = False):
        """``parallel_runtime``: the launch's peer-memory data plane (``parallel.runtime.ParallelRuntime``);
        its status word is checked once per step, before the optimizer.  ``lockstep_model_calls``:
        every rank issues the same number of model calls per window (expert parallelism: dispatch and
        combine are collectives), so locally degenerate groups are scored and trained with their zero
        advantages instead of being skipped."""
        config.validate()
        self.parallel_runtime = parallel_runtime
        self.lockstep_model_calls = bool(lockstep_model_calls)
        self.config = config
        self.policy = policy
        self.tokenizer = tokenizer
        self.reward_fn = reward_fn
        self.samples = list(samples)
        if not self.samples:
            raise TrainerError("no training samples")
        self.comm = comm or SoloComm()
        if topology not in ("dp", "tp"):
            raise TrainerError("topology must be 'dp' or 'tp'")
        self.topology = topology
        config.validate_reward_group_world(self.dp_world)
        if topology == "tp" and config.reward_group_scope != RewardGroupScope.LOCAL:
            raise TrainerError("distributed same-prompt reward groups need a data-parallel launch")
        self.run_dir = run_dir
        self.binding = binding
        self.metrics_writer = MetricsWriter(run_dir.metrics_path) if run_dir and self.is_writer else None
        self.candidate_writer = candidate_writer
        self.params = policy.trainable_params()
        if not self.params:
            raise TrainerError("the policy exposes no trainable tensors")
        uses_kl = config.beta > 0 or config.beta_schedule is not None
        if uses_kl and policy.lora_recipe() == "full_ft":
            # the KL reference is "this model with its adapters switched off"; with every base tensor
            # trainable there is no frozen reference left, and the penalty would silently be zero
            raise TrainerError("a KL penalty (beta > 0) needs a frozen reference policy; full fine-tuning has none")
        self.opt = FerrlAdamW(self.params, AdamWParams(config.lr, config.adam_beta1, config.adam_beta2, adam_eps,
                                                       config.weight_decay))
        self.fused_dp_step = fused_dp_step
        self.preempt_flag = threading.Event()
        self.must_discard = False
        self.history: list[Metrics] = []
        self.fuse_logp_old = config.mu == 1
        self.on_step_end: Optional[Callable[[int, Metrics], None]] = None
        self.fault_hook: Optional[Callable[[str], None]] = None  # host-side fault injection for tests
        self._timer: Optional[PhaseTimer] = None

    # ------------------------------------------------------------ topology
    @property
    def dp_world(self) -> int:
        return self.comm.world_size if self.topology == "dp" else 1

    @property
    def dp_rank(self) -> int:
        return self.comm.rank if self.topology == "dp" else 0

    @property
    def is_writer(self) -> bool:
        return self.comm.rank == 0

    def with_preemption_flag(self, flag: threading.Event) -> "Trainer":
        self.preempt_flag = flag
        return self

    def _fault(self, point: str):
        if self.fault_hook is not None:
            self.fault_hook(point)

    # ----------------------------------------------------------- selection
    def select_prompt(self, step: int, slot: int) -> PromptSelection:
        """Prompt for accumulation ``slot`` of window ``step``. Windows consume
        prompts contiguously; rank ``r`` takes the slice at offset ``r*slots``."""
        c = self.config
        slots = c.grad_accum_steps * c.prompts_per_item
        world, rank = self.dp_world, self.dp_rank
        n = len(self.samples)
        if c.reward_group_scope == RewardGroupScope.LOCAL:
            local = rank * slots + slot
            pi = step * slots * world + local
            return PromptSelection(pi % n, pi, pi * c.group_size)
        pi = step * slots + slot
        shard = step * slots * world + rank * slots + slot
        return PromptSelection(pi % n, pi, shard * c.group_size)

    def gen_config(self) -> GenConfig:
        c = self.config
        return GenConfig(c.group_size, c.max_new_tokens, c.temperature, c.eos_token_id, None, c.top_p)

    # ---------------------------------------------------------- collection
    def collect_groups(self, sels: Sequence[PromptSelection]) -> list[CollectedGroup]:
        c = self.config
        samples = [self.samples[s.sample_idx] for s in sels]
        prompt_ids = [list(self.tokenizer.encode(s.prompt)) for s in samples]
        if self.topology == "tp" and self.comm.world_size > 1:
            blob = repr([(p, s.rollout_global_row_base) for p, s in zip(prompt_ids, sels)]).encode()
            self.comm.require_consensus(blob, "rollout request")
        gen = self.gen_config()
        self._phase("rollout")
        self._fault("before_generate")
        rollouts = self.policy.generate_batch(prompt_ids, gen, [s.rollout_global_row_base for s in sels])
        self._phase_end("rollout")
        groups = []
        self._phase("reward")
        for sel, sample, pids, r in zip(sels, samples, prompt_ids, rollouts):
            try:
                validate_generated_rollout_semantics(r, pids, gen)
            except ValueError as e:
                raise TrainerError(f"policy returned a malformed rollout: {e}") from e
            completions = [self.tokenizer.decode(r.completion(i)) for i in range(len(r))]
            outcomes = self._rewards(sample, completions)
            rewards = [float(o.reward) for o in outcomes]
            mask = length_mask(r)
            truncated = mask_truncated_rows(r, c.eos_token_id, mask) if c.truncation_masking else 0
            groups.append(CollectedGroup(sel, sample, pids, r, completions, rewards, outcomes, [], mask, truncated,
                                         int(sum(r.completion_lens))))
        self._phase_end("reward")
        return groups

    def _rewards(self, sample: Sample, completions: list):
        """Rank 0 of a tensor-parallel group owns the verifier; peers receive the
        values in one broadcast (the reference all-reduces one scalar per reward)."""
        from .rewards import RewardOutcome
        if self.topology == "tp" and self.comm.world_size > 1:
            import json
            blob = None
            if self.comm.rank == 0:
                try:
                    out = self.reward_fn.reward_group_detailed(sample, completions)
                    blob = json.dumps({"ok": [[o.reward, o.diagnostic, o.metadata] for o in out]}).encode()
                except Exception as e:  # noqa: BLE001 - shipped to peers as a coordinated failure
                    blob = json.dumps({"err": repr(e)}).encode()
            d = json.loads(self.comm.broadcast_bytes(blob, 0).decode())
            if "err" in d:
                raise TrainerError(f"reward function failed on rank 0: {d['err']}")
            return [RewardOutcome(*o) for o in d["ok"]]
        try:
            out = self.reward_fn.reward_group_detailed(sample, completions)
        except RewardError:
            raise
        if len(out) != len(completions):
            raise TrainerError("reward function returned a different number of rewards than completions")
        return out

    def _advantages(self, groups: list[CollectedGroup]) -> None:
        c = self.config
        scale = ScaleRewards(c.scale_rewards)
        if c.reward_group_scope == RewardGroupScope.LOCAL or self.dp_world == 1:
            for g in groups:
                g.advantages = grpo.group_advantages(g.rewards, scale)
            return
        # distributed same-prompt: every rank holds a shard of the SAME group;
        # gather all shards' rewards and normalise with the global moments.
        import struct
        flat = [r for g in groups for r in g.rewards]
        blobs = self.comm.all_gather_bytes(struct.pack(f"<{len(flat)}d", *flat))
        per_rank = [struct.unpack(f"<{len(b) // 8}d", b) for b in blobs]
        off = 0
        for g in groups:
            n = len(g.rewards)
            allr = [v for pr in per_rank for v in pr[off:off + n]]
            m = grpo.finite_moments(allr)
            g.advantages = grpo.advantages_from_moments(g.rewards, m.mean, m.sample_std(), scale)
            off += n

    # ------------------------------------------------------- materialise
    def materialize(self, groups: list[CollectedGroup], beta: float, stats: WindowStats) -> Optional[LiveItem]:
        c = self.config
        dev = self.policy.device()
        for g in groups:
            stats.groups += 1
            stats.rows += len(g.rollout)
            stats.rewards += g.rewards
            m = grpo.finite_moments(g.rewards)
            stats.group_stds.append(m.sample_std())
            stats.zero_std_groups += int(m.sample_std() == 0.0)
            stats.truncated += g.truncated
            stats.completion_tokens += g.completion_tokens
            stats.completion_len_max = max(stats.completion_len_max, max(g.rollout.completion_lens))
            stats.dropped_rows += grpo.zero_mask_rows(g.mask.tolist()) if g.truncated else 0
        live = [g for g in groups if g.live or beta > 0.0 or self.lockstep_model_calls]
        stats.live_groups += len(live)
        if not live:
            return None
        rollouts = [g.rollout for g in live]
        adv = torch.tensor([a for g in live for a in g.advantages], dtype=torch.float32, device=dev)
        mask = torch.cat([g.mask for g in live]).to(dev)
        have_lp = all(r.rollout_logprobs is not None for r in rollouts)
        rlp = torch.cat([r.rollout_logprobs for r in rollouts]).to(dev) if have_lp else None
        logp_old = None
        tis_w = None
        if not self.fuse_logp_old:
            self._phase("logp_old")
            logp_old = self.policy.token_logprobs_detached(rollouts).detach()
            self._phase_end("logp_old")
            if rlp is not None:
                tis_w = self._rollout_ratio(logp_old, rlp, mask, stats)
        logp_ref = None
        if beta > 0.0:
            self._phase("logp_ref")
            was = self.policy.adapter_enabled()
            self.policy.set_adapter_enabled(False)
            try:
                logp_ref = self.policy.token_logprobs_detached(rollouts).detach()
            finally:
                self.policy.set_adapter_enabled(was)
            self._phase_end("logp_ref")
        return LiveItem(rollouts, adv, mask, logp_old, logp_ref, tis_w, rlp)

    def _rollout_ratio(self, logp_old, rlp, mask, stats: WindowStats) -> Optional[torch.Tensor]:
        """Scoring-vs-rollout importance ratio telemetry and (optionally) the
        truncated-importance-sampling weights (reference trainer.rs:9335-9410)."""
        c = self.config
        keep = mask > 0
        lr = torch.where(keep, logp_old - rlp, torch.zeros_like(logp_old))
        ratio = lr.exp()
        n = float(keep.sum().item())
        if n > 0:
            stats.ratio_sum += float((ratio * keep).sum().item())
            stats.logratio_sum += float(lr.sum().item())
            stats.ratio_max = max(stats.ratio_max, float(torch.where(keep, ratio, torch.zeros_like(ratio)).max().item()))
            stats.ratio_capped += float(((ratio > c.tis_imp_ratio_cap) & keep).sum().item())
            stats.ratio_tokens += n
        if not c.tis:
            return None
        return torch.where(keep, ratio.clamp(max=c.tis_imp_ratio_cap), torch.ones_like(ratio)).detach()

    # --------------------------------------------------------------- update
    def _item_backward(self, item: LiveItem, window_tokens: float, beta: float, stats: WindowStats, agg: dict):
        c = self.config
        G = c.group_size
        rows_total = sum(len(r) for r in item.rollouts)
        mb = c.backward_microbatch_size if c.backward_microbatch_size > 0 else rows_total
        global_slots = c.grad_accum_steps * c.prompts_per_item * self.dp_world
        lt = LossType(c.loss_type)
        # flatten to row-sliced rollouts
        flat = []
        for r in item.rollouts:
            for s in range(0, len(r), mb):
                e = min(len(r), s + mb)
                flat.append((r, s, e))
        # merge consecutive slices up to mb rows
        batches, cur, cur_n = [], [], 0
        for r, s, e in flat:
            if cur and cur_n + (e - s) > mb:
                batches.append(cur)
                cur, cur_n = [], 0
            cur.append((r, s, e))
            cur_n += e - s
        if cur:
            batches.append(cur)
        row0 = 0
        for b in batches:
            subs = [Rollout(r.token_ids[s:e], r.prompt_len, r.completion_lens[s:e],
                            None if r.rollout_logprobs is None else r.rollout_logprobs[s:e]) for r, s, e in b]
            n = sum(len(s) for s in subs)
            sl = slice(row0, row0 + n)
            row0 += n
            self._phase("forward")
            logp = self.policy.token_logprobs(subs)
            self._phase_end("forward")
            mask, adv = item.mask[sl], item.advantages[sl]
            tis_w = None if item.tis_w is None else item.tis_w[sl]
            if item.logp_old is None:
                logp_old = logp.detach()
                if item.rollout_lp is not None and agg["epoch"] == 0:
                    tis_w = self._rollout_ratio(logp_old, item.rollout_lp[sl], mask, stats)
            else:
                logp_old = item.logp_old[sl]
            ref = None if item.logp_ref is None else item.logp_ref[sl]
            scale = 1.0 if lt is LossType.DAPO else n / float(G * global_slots)
            cfg = LossConfig(c.clip_eps, c.clip_eps_high_eff(), beta, lt,
                             ImportanceSamplingLevel(c.importance_sampling_level), window_tokens, scale)
            loss = grpo.grpo_loss(logp, logp_old, ref, adv, mask, cfg, tis_w)
            st = grpo.loss_stats(logp.detach(), logp_old, ref, adv, mask, cfg)
            agg["kl"] += st.kl_sum
            agg["clip_low"] += st.clip_low_sum
            agg["clip_high"] += st.clip_high_sum
            agg["tokens"] += st.token_count
            agg["loss"] += float(loss.detach().item())
            self._phase("backward")
            self._fault("before_backward")
            self.policy.backward(loss)
            self._phase_end("backward")

    def accumulate_step(self, live: list[LiveItem], window_tokens: float, beta: float, lr: float,
                        stats: WindowStats, agg: dict) -> None:
        if self.fused_dp_step is not None:
            self.fused_dp_step.prepare_grads()   # .grad tensors are views of the peer-visible flat buffer
        else:
            for p in self.params:
                p.grad = None
        def local_backward():
            for item in live:
                self._item_backward(item, window_tokens, beta, stats, agg)
        # every rank must have finished (or failed) its local backward before anyone enters the
        # gradient collective; a failure anywhere raises on all ranks here, not at a timeout.
        # The fused peer-memory step already sums an "uncovered" count over the world on the device and
        # skips the update when it is non-zero, so there a failed backward rides on that count and the
        # healthy step has no rendezvous of its own.
        backward_error = None
        if self.fused_dp_step is not None and self.parallel_runtime is None and self._deferred_agreement():
            try:
                local_backward()
            except CommError:
                raise
            except Exception as e:  # noqa: BLE001 - reported to every rank through the fused step's count
                backward_error = e
        else:
            self._rendezvous(local_backward, "backward")
        if self.parallel_runtime is not None:
            # a bounded peer wait that ran out inside a fused tensor-/expert-parallel kernel leaves a
            # status word behind: raise CommTimeout here, before the optimizer touches anything
            self._rendezvous(lambda: self.parallel_runtime.check("tensor-/expert-parallel kernels of this step"),
                             "peer-memory status")
        self._phase("grad_reduce_optimizer")
        world = self.comm.world_size
        if self.fused_dp_step is not None:
            missing = self.fused_dp_step.missing() if live else []
            nonfinite = []                       # counted inside the kernel, world-wide
        else:
            # a rank with live items but an absent gradient is a coverage failure; a rank with no live
            # item simply contributes zeros.  Either way every slot is materialised with zeros so that
            # all ranks enter the same tensor collective with the same shapes, and the failure is
            # reported through the uncovered count on every rank (reference trainer.rs
            # materialize_zero_grad_slots + reduce_accumulated_grads).
            missing, nonfinite = grad_coverage(self.params)
            if not live:
                missing = []
            for p in self.params:
                if p.grad is None:
                    p.grad = torch.zeros_like(p)
        uncovered = float(len(missing) + len(nonfinite))
        if self.fused_dp_step is not None:
            # fused peer-memory path: all-reduce + clip + AdamW in one pass
            self.opt.set_learning_rate(lr)
            if backward_error is not None:
                uncovered = PEER_FAILED_COUNT
            res = self.fused_dp_step(self.opt, [p.grad for p in self.params], self.config.max_grad_norm, uncovered)
            agg["grad_norm"] = res.grad_norm
            if backward_error is not None:
                raise PeerFailure(f"backward failed on this rank: {backward_error!r}", local=backward_error)
            if res.uncovered >= PEER_FAILED_COUNT:
                raise PeerFailure("backward failed on a peer rank", local=None)
            if res.uncovered > 0:
                raise GradCoverageError(f"{int(res.uncovered)} trainable tensor(s) uncovered or non-finite "
                                        "somewhere in the world")
            agg["stepped"] = res.stepped
            self._phase_end("grad_reduce_optimizer")
            if res.stepped:
                self.policy.on_params_updated()
            return
        if world > 1:
            self.comm.all_reduce_sum([p.grad for p in self.params])
            uncovered = self.comm.all_reduce_scalar_sum(uncovered)
        if uncovered > 0:
            raise GradCoverageError(
                f"gradient coverage failure: missing={missing} non_finite={nonfinite} (world total {int(uncovered)})")
        grads = [p.grad for p in self.params]
        norm = global_grad_norm(grads)
        agg["grad_norm"] = norm
        if norm == 0.0:
            agg["stepped"] = False  # all-zero gradient: skip, keep Adam state untouched
            self._phase_end("grad_reduce_optimizer")
            return
        gscale = 1.0
        if self.config.max_grad_norm is not None and norm > self.config.max_grad_norm:
            gscale = self.config.max_grad_norm / norm
        self.opt.set_learning_rate(lr)
        self._fault("before_optimizer")
        self.opt.step(grads, gscale)
        agg["stepped"] = True
        self.policy.on_params_updated()
        self._phase_end("grad_reduce_optimizer")

    # ---------------------------------------------------------------- window
    def collect_window(self, step: int, defer_agreement: bool = False) -> list:
        """Rollout + reward half of a window: ``[(accum_index, [CollectedGroup, ...]), ...]``.
        ``defer_agreement``: the caller's next exchange reports a failure of this stage (``run_window``)."""
        c = self.config
        P = c.prompts_per_item
        def local():
            out = []
            for j in range(c.grad_accum_steps):
                sels = [self.select_prompt(step, j * P + q) for q in range(P)]
                out.append((j, self.collect_groups(sels)))
            return out
        # rollout + rewards touch no data-parallel collective.  With rank-local advantages nothing
        # between here and the window-size exchange needs the peers, so a failure is carried to that
        # exchange instead of a rendezvous of its own; cross-rank normalisation needs agreement first.
        if defer_agreement and self._deferred_agreement():
            out = self._stage(local, "rollout collection")
            if out is None:
                return []
        else:
            out = self._rendezvous(local, "rollout collection")
        for _, groups in out:
            self._advantages(groups)
        return out

    def run_window(self, step: int, lr: float, beta: float, collected: Optional[list] = None) -> tuple[Metrics, int]:
        c = self.config
        stats = WindowStats()
        live: list[LiveItem] = []
        all_groups: list[CollectedGroup] = []
        self._pending_failure = None
        if collected is None:
            collected = self.collect_window(step, defer_agreement=True)

        def local_materialize():
            for j, groups in collected:
                all_groups.extend(groups)
                item = self.materialize(groups, beta, stats)
                if item is not None:
                    live.append(item)
        if self._deferred_agreement():
            # one exchange carries the window size, the live-item count and whether any rank failed in
            # the rollout or scoring stage: a healthy step has no other rendezvous before its backward
            self._stage(local_materialize, "rollout scoring")
            failed = self._pending_failure
            self._pending_failure = None
            local_tokens = stats.completion_tokens
            window_tokens, n_live, failures = self.comm.all_reduce_scalars_sum(
                [float(local_tokens), float(len(live)), 0.0 if failed is None else 1.0])
            if failures > 0:
                if failed is not None:
                    raise PeerFailure(f"{failed[0]} failed on this rank: {failed[1]!r}", local=failed[1])
                raise PeerFailure(f"rollout or scoring failed on {int(failures)} peer rank(s)", local=None)
            if c.candidate_log_top_k > 0 and self.candidate_writer is not None:
                self._log_candidates(step, all_groups)
        else:
            self._rendezvous(local_materialize, "rollout scoring")
            if c.candidate_log_top_k > 0 and self.candidate_writer is not None:
                self._log_candidates(step, all_groups)
            local_tokens = stats.completion_tokens
            window_tokens, n_live = self.comm.all_reduce_scalars_sum([float(local_tokens), float(len(live))]) \
                if self.topology == "dp" else (float(local_tokens), float(len(live)))
        window_tokens = max(window_tokens, 1.0)
        agg = {"kl": 0.0, "clip_low": 0.0, "clip_high": 0.0, "tokens": 0.0, "loss": 0.0, "grad_norm": 0.0,
               "stepped": False, "epoch": 0}
        if n_live > 0:
            for e in range(c.mu):
                agg["epoch"] = e
                self.accumulate_step(live, window_tokens, beta, lr, stats, agg)
        elif self.parallel_runtime is not None:
            # no update this window: the rollout and scoring kernels still ran over peer memory
            self._rendezvous(lambda: self.parallel_runtime.check("tensor-/expert-parallel kernels of this step"),
                             "peer-memory status")
        return self._build_metrics(step, lr, beta, stats, agg), local_tokens

    def _build_metrics(self, step, lr, beta, stats: WindowStats, agg: dict) -> Metrics:
        m = Metrics(step=step, lr=lr, beta=beta, rank=self.comm.rank, world_size=self.comm.world_size)
        if stats.rewards:
            mom = grpo.finite_moments(stats.rewards)
            m.reward_mean, m.reward_std = mom.mean, mom.population_std()
        m.frac_reward_zero_std = stats.zero_std_groups / max(stats.groups, 1)
        m.frac_truncated = stats.truncated / max(stats.rows, 1)
        m.completion_len = stats.completion_tokens / max(stats.rows, 1)
        m.completion_len_max = float(stats.completion_len_max)
        m.dropped_rows = stats.dropped_rows
        m.live_groups = stats.live_groups
        m.skipped_groups = stats.groups - stats.live_groups
        sums = [agg["kl"], agg["clip_low"], agg["clip_high"], agg["tokens"], agg["loss"]]
        if self.topology == "dp" and self.comm.world_size > 1:
            sums = self.comm.all_reduce_scalars_sum(sums)
        tok = max(sums[3], 1.0)
        m.kl = sums[0] / tok
        m.clip_ratio_low, m.clip_ratio_high = sums[1] / tok, sums[2] / tok
        m.clip_ratio = m.clip_ratio_low + m.clip_ratio_high
        m.loss = sums[4]
        m.grad_norm = agg["grad_norm"]
        if stats.ratio_tokens > 0:
            m.rollout_ratio_mean = stats.ratio_sum / stats.ratio_tokens
            m.rollout_logratio_mean = stats.logratio_sum / stats.ratio_tokens
            m.rollout_ratio_max = stats.ratio_max
            m.frac_rollout_ratio_capped = stats.ratio_capped / stats.ratio_tokens
            m.rollout_capture_tokens = int(stats.ratio_tokens)
        return m

    def _log_candidates(self, step: int, groups: list[CollectedGroup]) -> None:
        k = self.config.candidate_log_top_k
        rows = []
        for g in groups:
            for i, (rw, comp) in enumerate(zip(g.rewards, g.completions)):
                rows.append((rw, g, i, comp))
        rows.sort(key=lambda t: (-t[0], t[1].selection.prompt_index, t[2]))
        for rw, g, i, comp in rows[:k]:
            o = g.outcomes[i]
            self.candidate_writer.append(CandidateRecord(
                step=step, rank=self.comm.rank, world_size=self.comm.world_size,
                prompt_index=g.selection.prompt_index, group_index=i, reward=rw,
                completion_len_tokens=g.rollout.completion_lens[i], completion=comp,
                reward_diagnostic=o.diagnostic, reward_metadata=o.metadata))

    def _rendezvous(self, fn, what: str):
        """Run a rank-local stage, then agree on its outcome across data-parallel ranks."""
        if self.topology == "dp" and self.comm.world_size > 1:
            return self.comm.coordinate(fn, what)
        return fn()

    _pending_failure = None

    def _deferred_agreement(self) -> bool:
        """True when the rollout and scoring stages need no rendezvous of their own: plain data
        parallelism (no lockstep model calls) with rank-local advantage normalisation."""
        return (self.topology == "dp" and self.comm.world_size > 1 and not self.lockstep_model_calls
                and (self.config.reward_group_scope == RewardGroupScope.LOCAL or self.dp_world == 1))

    def _stage(self, fn, what: str):
        """Run a rank-local stage whose outcome the ranks agree on at the window's next exchange; after
        a failure the later stages of this rank are skipped (``None``) until that exchange."""
        if self._pending_failure is not None:
            return None
        try:
            return fn()
        except CommError:
            raise
        except Exception as e:  # noqa: BLE001 - reported to every rank at the next exchange
            self._pending_failure = (what, e)
            return None

    # ------------------------------------------------------------ phases
    def _phase(self, label: str):
        if self._timer is not None:
            self._timer.start(label)
        if self._probe is not None:
            self._probe.record(label + "_start")

    def _phase_end(self, label: str):
        if self._timer is not None:
            self._timer.stop(label)
        if self._probe is not None:
            self._probe.record(label + "_end")

    _probe: Optional[GpuMemoryProbe] = None

    # ------------------------------------------------------------ rollback
    def _snapshot(self):
        """Pre-window copy of adapters, Adam moments and sampler state for rollback (reference
        trainer.rs:5120-5290).  The copies live in three persistent buffer lists refilled with one
        multi-tensor copy each (three launches per step instead of one clone per tensor)."""
        cur = [p.detach() for p in self.params]
        bufs = getattr(self, "_snap_bufs", None)
        if bufs is None or len(bufs[0]) != len(cur) or any(b.shape != c.shape or b.device != c.device
                                                          for b, c in zip(bufs[0], cur)):
            bufs = ([torch.empty_like(c) for c in cur], [torch.empty_like(t) for t in self.opt.m],
                    [torch.empty_like(t) for t in self.opt.v])
            self._snap_bufs = bufs
        with torch.no_grad():
            if cur:
                torch._foreach_copy_(bufs[0], cur)
                torch._foreach_copy_(bufs[1], list(self.opt.m))
                torch._foreach_copy_(bufs[2], list(self.opt.v))
        return (bufs[0], OptimizerState(self.opt.step_t, bufs[1], bufs[2]), self.policy.sampler_state())

    def check_replicated_adapters(self) -> None:
        """Tensor parallelism keeps every adapter replicated: all ranks must hold bit-identical values,
        or their gradients (summed over the group) update diverging copies.  The reference proves it by
        all-reducing every adapter value on each backward (gemma4.rs:157-274); here each rank reduces its
        adapters to two float64 moments per tensor on the device and the ranks compare one digest."""
        if self.topology != "tp" or self.comm.world_size == 1 or not self.params:
            return
        with torch.no_grad():
            flat = [p.detach().double() for p in self.params]
            fp = torch.stack([t.sum() for t in flat] + [(t * t).sum() for t in flat]).cpu()
        self.comm.require_consensus(fp.numpy().tobytes(), "replicated adapter values")

    def _restore(self, snap) -> None:
        try:
            vals, ost, sst = snap
            with torch.no_grad():
                for p, v in zip(self.params, vals):
                    p.copy_(v)
            self.opt.load_state(ost)
            self.policy.restore_sampler_state(sst)
            self.policy.on_params_updated()
        except Exception as e:  # noqa: BLE001
            self.must_discard = True
            raise MustDiscard(f"rollback failed, trainer state is undefined: {e}") from e

    # ---------------------------------------------------------------- step
    def step(self, step: int) -> Metrics:
        """Run optimizer step ``step`` end to end and return its metrics row.
        Under data parallelism a failure on any rank rolls every rank back to
        the pre-window state and raises on all of them."""
        if self.must_discard:
            raise MustDiscard("trainer must be discarded after a failed rollback")
        c = self.config
        lr, beta = c.lr_at(step), c.beta_at(step)
        dev = self.policy.device()
        self._timer = PhaseTimer(dev)
        self._probe = GpuMemoryProbe(c.gpu_memory_probe, dev if dev.type == "cuda" else None)
        self.check_replicated_adapters()
        snap = self._snapshot() if self.comm.world_size > 1 or self.fault_hook is not None else None
        cand_mark = self.candidate_writer.mark() if self.candidate_writer is not None else None
        t0 = time.perf_counter()
        wait0 = float(getattr(self.comm, "wait_s", 0.0))
        try:
            m, local_tokens = self.run_window(step, lr, beta)
        except CommError:
            raise                      # communicator failures are terminal: no rollback collective is possible
        except Exception:
            if cand_mark is not None:
                self.candidate_writer.rollback(cand_mark)   # the window's candidate rows go with its state
            if snap is not None:
                self._restore(snap)
            raise
        phases = self._timer.collect()
        m.step_secs = time.perf_counter() - t0
        m.tokens_per_sec = local_tokens / m.step_secs if m.step_secs > 0 else 0.0
        m.phase_ms = {k: round(v, 3) for k, v in phases.items()}
        if self.comm.world_size > 1:
            # host time blocked inside collectives during this step: the wait for the slowest rank at each
            # agreement point plus the exchanges themselves (it overlaps the device phases above)
            m.phase_ms["comm_wait"] = round(1e3 * (float(getattr(self.comm, "wait_s", 0.0)) - wait0), 3)
        if self._probe.enabled:
            m.cuda_mem_start_used_bytes, m.cuda_mem_peak_used_bytes = self._probe.start, self._probe.peak
            m.cuda_mem_end_used_bytes, m.cuda_mem_total_bytes = self._probe.end, self._probe.total
            m.cuda_mem_peak_delta_bytes = max(0, int(self._probe.peak) - int(self._probe.start))
            m.cuda_mem_probe_events = self._probe.events
        m.decoder_cache_bytes = int(getattr(self.policy, "last_cache_bytes", 0))
        self.history.append(m)
        if self.metrics_writer is not None:
            self.metrics_writer.append(m)
        return m

    # ----------------------------------------------------------------- run
    def train(self, start_step: int = 0) -> RunStop:
        c = self.config
        self._prepare()
        for step in range(start_step, c.steps):
            m = self.step(step)
            log.info("step %d reward %.4f loss %.5f kl %.5f grad %.4f tok/s %.1f", step, m.reward_mean, m.loss,
                     m.kl, m.grad_norm, m.tokens_per_sec)
            if self.on_step_end is not None:
                self.on_step_end(step, m)
            done = step + 1
            if c.checkpoint_every is not None and done % c.checkpoint_every == 0 and done < c.steps:
                self.write_checkpoint(done)
            if self._poll_preempt():
                if not self._has_checkpoint(done):
                    self.write_checkpoint(done)
                return RunStop.PREEMPTED
        if c.checkpoint_every is not None and not self._has_checkpoint(c.steps):
            self.write_checkpoint(c.steps)
        return RunStop.COMPLETED

    def _prepare(self) -> None:
        """Launch consensus: trainer config and optimizer tensor schema must be
        identical on every rank (reference trainer.rs:7051-7119)."""
        if self.comm.world_size > 1:
            self.comm.require_consensus(self.config.digest().encode(), "trainer config")
            self.comm.require_consensus(repr(self.opt.schema()).encode(), "optimizer tensor schema")
            self.comm.require_consensus(self.policy.sampler_state(), "sampler state")

    def _poll_preempt(self) -> bool:
        flag = 1.0 if self.preempt_flag.is_set() else 0.0
        if self.comm.world_size > 1:
            flag = self.comm.all_reduce_scalar_sum(flag)
        return flag > 0

    # ------------------------------------------------ separated collector / learner
    def collect_to_ledger(self, step: int, writer) -> "object":
        """Collector side: roll out and score window ``step`` and persist it; no update.
        Under data parallelism every rank stages its shard and rank 0 commits the manifest
        once all shards exist (reference trainer.rs:2211-2679, rollout_ledger.rs:676-1110)."""
        from . import ledger as L
        c = self.config
        collected = self.collect_window(step)
        cap = L.f64_bits(c.tis_imp_ratio_cap) if c.tis else None
        ctl = L.LedgerControls(c.grad_accum_steps, c.prompts_per_item, c.group_size, c.max_new_tokens,
                               c.reward_group_scope, c.scale_rewards, c.eos_token_id, c.truncation_masking,
                               L.f64_bits(c.lr_at(step)), L.f64_bits(c.beta_at(step)), cap)
        groups = [L.LedgerGroup.from_collected(j, g) for j, gs in collected for g in gs]
        tokens = sum(g.completion_tokens for _, gs in collected for g in gs)
        st = L.LedgerStep(step, self.dp_rank, self.dp_world, ctl, tokens,
                          sum(1 for _, gs in collected for g in gs if g.live), list(self.policy.sampler_state()), groups)
        if self.comm.world_size == 1:
            writer.write_step(st)
            return st
        if self.topology == "tp":
            # every tensor-parallel rank holds the same window: it is one artifact, written by rank 0
            self.comm.coordinate(lambda: writer.write_step(st) if self.is_writer else None, "ledger write")
            return st
        # rank 0 draws the stage nonce and creates the hidden stage; every rank writes its shard
        # into it; the outcome of each phase is agreed before anyone moves on, and the stage is
        # removed only after all ranks have stopped writing.
        import os as _os
        nonce = int.from_bytes(self.comm.broadcast_bytes(_os.urandom(8) if self.is_writer else None), "little")
        stage = self.comm.coordinate(lambda: writer.create_distributed_stage(step, nonce) if self.is_writer else None,
                                     "ledger stage creation")
        try:
            if not self.is_writer:
                stage = self.comm.coordinate(lambda: writer.open_distributed_stage(step, nonce), "ledger stage open")
            else:
                self.comm.coordinate(lambda: None, "ledger stage open")
            self.comm.coordinate(lambda: writer.write_distributed_shard(stage, st), "ledger shard write")
            self.comm.coordinate(lambda: writer.commit_distributed_stage(stage) if self.is_writer else None,
                                 "ledger commit")
        except PeerFailure:
            if self.is_writer and stage is not None:
                writer.abort_distributed_stage(stage)
            raise
        return st

    def train_from_ledger(self, record) -> Metrics:
        """Learner side: run the update of a previously collected window (this rank's shard)."""
        from . import ledger as L
        c = self.config
        if record.controls.group_size != c.group_size or record.controls.completion_width != c.max_new_tokens:
            raise TrainerError("ledger step was collected under different group_size / max_new_tokens")
        if record.world_size != self.dp_world or record.rank != self.dp_rank:
            raise TrainerError("ledger shard belongs to a different rank/world")
        if record.controls.tis_imp_ratio_cap_bits != (L.f64_bits(c.tis_imp_ratio_cap) if c.tis else None):
            raise TrainerError("ledger step was collected under a different truncated-importance-sampling cap")
        by_item: dict = {}
        for g in record.groups:
            r = g.rollout()
            sel = PromptSelection(g.prompt_index % len(self.samples), g.prompt_index, g.rollout_global_row_base)
            cg = CollectedGroup(sel, self.samples[sel.sample_idx], list(g.prompt_token_ids), r, [], g.rewards(), [],
                                g.advantages(), g.mask(), 0, int(sum(r.completion_lens)))
            by_item.setdefault(g.accum_index, []).append(cg)
        collected = sorted(by_item.items())
        lr, beta = L.bits_f64(record.controls.effective_lr_bits), L.bits_f64(record.controls.effective_beta_bits)
        dev = self.policy.device()
        self._timer = PhaseTimer(dev)
        self._probe = GpuMemoryProbe(False)
        t0 = time.perf_counter()
        m, local_tokens = self.run_window(record.step, lr, beta, collected)
        m.phase_ms = self._timer.collect()
        m.step_secs = time.perf_counter() - t0
        m.tokens_per_sec = local_tokens / m.step_secs if m.step_secs > 0 else 0.0
        self.policy.restore_sampler_state(bytes(record.post_rollout_sampler_state))
        self.history.append(m)
        if self.metrics_writer is not None:
            self.metrics_writer.append(m)
        return m

    # ------------------------------------------------ collector / learner chain
    def learner_semantic_config_sha256(self) -> str:
        """Digest of the trainer configuration without the operational fields (run horizon, checkpoint
        cadence, candidate logging, memory probing) that do not change one learner update."""
        from .config import canonical_digest
        d = self.config.to_json()
        for k in ("steps", "checkpoint_every", "candidate_log_top_k", "gpu_memory_probe"):
            d.pop(k, None)
        return canonical_digest(d, b"ferrl-b200/trainer-config-learner/v1")

    def ledger_identity(self, step: int, lineage: Optional[str] = None):
        """The identity a window collected NOW, for ``step``, must carry: digests of this trainer's
        configuration, frozen policy, adapter values, optimizer moments and sampler state."""
        from . import ledger as L
        dg = L.state_digests(self.params, self.opt, self.policy.sampler_state(), self.policy.lora_recipe())
        policy = self.binding.frozen_policy_sha256 if self.binding is not None else "0" * 64
        return L.LedgerIdentity(self.learner_semantic_config_sha256(), policy, dg["adapter_sha256"], dg["optimizer_sha256"],
                                dg["sampler_sha256"], step, self.opt.step_t, dg["tensor_schema_sha256"],
                                lineage or L.ROOT_LINEAGE)

    def collect_window_to(self, ledger_root: str, step: int, lineage: Optional[str] = None):
        """Collector: write window ``step`` under the identity of the current state."""
        from . import ledger as L
        w = L.RolloutLedgerWriter(ledger_root, self.ledger_identity(step, lineage), rank=self.dp_rank,
                                  world_size=self.dp_world)
        return self.collect_to_ledger(step, w)

    def learn_window_from(self, ledger_root: str, step: int, lineage: Optional[str] = None):
        """Learner: consume window ``step`` only if it was collected from exactly this state (identity
        and controls are checked before anything is mutated), apply the update and return the
        ``LedgerContinuation`` that the next collector builds on.  With a run directory the
        post-update state is also published as a no-replace continuation checkpoint."""
        from . import ledger as L
        lineage = lineage or L.ROOT_LINEAGE
        c = self.config
        want = self.ledger_identity(step, lineage)
        ctl = L.LedgerControls(c.grad_accum_steps, c.prompts_per_item, c.group_size, c.max_new_tokens,
                               c.reward_group_scope, c.scale_rewards, c.eos_token_id, c.truncation_masking, 0, 0,
                               L.f64_bits(c.tis_imp_ratio_cap) if c.tis else None)
        reader = L.RolloutLedgerReader(ledger_root, want, ctl)
        record = reader.read_step(step, rank=self.dp_rank)
        consumed = reader.consumed_ledger_sha256(step)
        self.train_from_ledger(record)
        post = L.state_digests(self.params, self.opt, self.policy.sampler_state(), self.policy.lora_recipe())
        cont = L.LedgerContinuation(step + 1, want.policy_sha256, want.trainer_config_sha256, post["tensor_schema_sha256"],
                                    post["adapter_sha256"], post["optimizer_sha256"], post["sampler_sha256"], lineage,
                                    consumed, L.lineage_sha256(lineage, consumed, step + 1, post),
                                    world_size=self.comm.world_size if self.topology == "dp" else 1,
                                    tensor_parallel_world_size=self.comm.world_size if self.topology == "tp" else 1)
        if self.comm.world_size > 1:
            self.comm.require_consensus(cont.lineage_sha256.encode(), "rollout-ledger continuation lineage")
        if self.run_dir is not None and self.binding is not None:
            def write():
                if self.is_writer:
                    save_checkpoint(self.run_dir.checkpoints_dir, step + 1, [p.detach() for p in self.params],
                                    self.opt.state(), self.policy.sampler_state(), self.binding,
                                    world_size=self.comm.world_size, topology=self.topology,
                                    continuation=cont.to_json())
            if self.comm.world_size > 1:
                self.comm.coordinate(write, "continuation checkpoint write")
            else:
                write()
        return cont

    # ---------------------------------------------------------- checkpoints
    def _has_checkpoint(self, step: int) -> bool:
        import os
        from .checkpoint import step_dir
        return self.run_dir is not None and os.path.isdir(step_dir(self.run_dir.checkpoints_dir, step))

    def write_checkpoint(self, step: int) -> None:
        """Rank 0 writes; the outcome is agreed by all ranks before anyone proceeds."""
        if self.run_dir is None or self.binding is None:
            return

        def write():
            if self.is_writer:
                save_checkpoint(self.run_dir.checkpoints_dir, step, [p.detach() for p in self.params],
                                self.opt.state(), self.policy.sampler_state(), self.binding,
                                world_size=self.comm.world_size, topology=self.topology,
                                fault_hook=self.fault_hook)
        if self.comm.world_size > 1:
            self.comm.coordinate(write, "checkpoint write")
        else:
            write()

    def resume_latest(self) -> int:
        """Restore the newest complete checkpoint; returns the step to continue
        from (0 when none exists). Rank 0 scans; its decision - including a
        failure - is shared with every rank before any state is mutated."""
        import json
        if self.run_dir is None:
            return 0
        decision = None
        if self.is_writer:
            try:
                found = latest_checkpoint(self.run_dir.checkpoints_dir)
                decision = {"step": None if found is None else found[0]}
            except CheckpointError as e:
                decision = {"err": str(e)}
        if self.comm.world_size > 1:
            decision = json.loads(self.comm.broadcast_bytes(
                None if decision is None else json.dumps(decision).encode(), 0).decode())
        if "err" in decision:
            raise CheckpointMismatch(f"resume discovery failed on rank 0: {decision['err']}")
        if decision["step"] is None:
            return 0
        from .checkpoint import step_dir
        path = step_dir(self.run_dir.checkpoints_dir, decision["step"])

        def prepare() -> LoadedCheckpoint:
            lc = prepare_checkpoint(path, self.binding, [tuple(p.shape) for p in self.params],
                                    world_size=self.comm.world_size, topology=self.topology)
            if lc.manifest.sampler_bytes() is not None:
                self.policy.validate_sampler_state(lc.manifest.sampler_bytes())
            if lc.optimizer is not None:
                FerrlAdamW(self.params, self.opt.hp).load_state(lc.optimizer)  # throw-away preflight
            return lc
        lc = self.comm.coordinate(prepare, "checkpoint load") if self.comm.world_size > 1 else prepare()
        if self.comm.world_size > 1:
            self.comm.require_consensus(json.dumps(lc.manifest.to_json(), sort_keys=True).encode(),
                                        "checkpoint manifest")
        snap = self._snapshot()
        try:
            with torch.no_grad():
                for p, t in zip(self.params, lc.adapters):
                    p.copy_(t.to(p.dtype))
            if lc.optimizer is not None:
                self.opt.load_state(lc.optimizer)
            if lc.manifest.sampler_bytes() is not None:
                self.policy.restore_sampler_state(lc.manifest.sampler_bytes())
            self.policy.on_params_updated()
        except Exception:
            self._restore(snap)
            raise
        return int(lc.manifest.step)
