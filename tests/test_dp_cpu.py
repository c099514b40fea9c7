"""Distributed and full-model behaviour on CPU ranks (threads): liveness with degenerate shards,
durability under data parallelism, real-fixture lockstep in LoRA and full fine-tuning mode,
GSPO on the MoE fixture across a checkpoint boundary."""
import os

import pytest
import torch

from ferrl_b200.checkpoint import CheckpointBinding
from ferrl_b200.comm import run_ranks
from ferrl_b200.lm_policy import LmPolicy
from ferrl_b200.models.loader import LoaderOpts, load_auto_policy
from ferrl_b200.rewards import FnReward
from ferrl_b200.sampler import GrpoSampler
from ferrl_b200.telemetry import RunDir
from ferrl_b200.trainer import Trainer, TrainerError

from test_trainer_cpu import ListTok, cfg, echo_reward, make_policy, samples

FIX = os.path.join(os.path.dirname(__file__), "fixtures")


def varied(sample, completion):
    return float(sum(int(t) for t in completion.split()) % 3)


def fixture_policy(name, **kw):
    m = load_auto_policy(os.path.join(FIX, name), LoaderOpts(**kw))[0]
    return LmPolicy(m, GrpoSampler(11, 1.0))


def test_full_fine_tuning_moves_base_weights_and_refuses_a_kl_penalty():
    pol = fixture_policy("tiny_qwen35", full_ft=True)
    assert pol.lora_recipe() == "full_ft"
    before = [p.detach().clone() for p in pol.trainable_params()]
    tr = Trainer(pol, ListTok(), FnReward(varied), samples(), cfg(steps=2, lr=1e-3))
    tr.train()
    assert any(m.grad_norm > 0 for m in tr.history)
    moved = [not torch.equal(a, b.detach()) for a, b in zip(before, pol.trainable_params())]
    assert all(moved) and len(moved) > 20                              # embeddings, norms, projections: everything
    lora = fixture_policy("tiny_qwen35")
    assert len(lora.trainable_params()) != len(before) and lora.lora_recipe().startswith("lora:")
    with pytest.raises(TrainerError, match="frozen reference"):
        Trainer(fixture_policy("tiny_qwen35", full_ft=True), ListTok(), FnReward(varied), samples(), cfg(steps=1, beta=0.04))
    Trainer(lora, ListTok(), FnReward(varied), samples(), cfg(steps=1, beta=0.04))    # adapters keep a reference


@pytest.mark.parametrize("full_ft", [False, True])
def test_two_ranks_stay_in_bitwise_lockstep_on_the_hybrid_fixture(full_ft):
    def body(comm):
        tr = Trainer(fixture_policy("tiny_qwen35", full_ft=full_ft), ListTok(), FnReward(varied), samples(),
                     cfg(steps=2, prompts_per_item=1, lr=1e-3), comm=comm)
        tr.train()
        return [p.detach().clone() for p in tr.params], [m.grad_norm for m in tr.history]
    a, b = run_ranks(2, body, timeout=120)
    assert a[1] == b[1] and any(g > 0 for g in a[1])
    assert all(torch.equal(x, y) for x, y in zip(a[0], b[0]))


def test_moe_gspo_matches_across_a_checkpoint_boundary(tmp_path):
    """Sequence-level importance sampling on the sparse-MoE hybrid: stop after one step, resume in a
    fresh process image, and end bit-identical to the uninterrupted run."""
    gspo = dict(importance_sampling_level="sequence", lr=1e-3, checkpoint_every=1)
    binding = CheckpointBinding("a" * 64, "b" * 64, None)

    def trainer(steps, rd):
        pol = fixture_policy("tiny_qwen35_moe")
        b = CheckpointBinding(binding.frozen_policy_sha256, binding.trainer_config_sha256, pol.lora_recipe())
        return Trainer(pol, ListTok(), FnReward(varied), samples(), cfg(steps=steps, **gspo), run_dir=rd, binding=b)
    straight = trainer(2, RunDir.create(str(tmp_path / "a"), "r"))
    straight.train()
    assert any(m.grad_norm > 0 for m in straight.history)
    trainer(1, RunDir.create(str(tmp_path / "b"), "r")).train()
    resumed = trainer(2, RunDir.open(str(tmp_path / "b" / "r")))
    assert resumed.resume_latest() == 1
    resumed.train(1)
    for p, q in zip(straight.params, resumed.params):
        assert torch.equal(p.detach(), q.detach())


def test_degenerate_local_shard_still_joins_and_globally_degenerate_window_is_skipped():
    """Rank 1's rewards are constant (zero advantages, no local gradient) yet it joins every
    collective and ends with rank 0's update; when every rank is degenerate nobody steps."""
    def body(comm, both=False):
        flat = both or comm.rank == 1
        reward = FnReward((lambda s, c: 1.0) if flat else varied)
        tr = Trainer(make_policy(), ListTok(), reward, samples(), cfg(steps=2, prompts_per_item=1), comm=comm)
        tr.train()
        return [p.detach().clone() for p in tr.params], [m.grad_norm for m in tr.history], tr.opt.step_t
    a, b = run_ranks(2, body, timeout=60)
    assert a[1] == b[1] and any(g > 0 for g in a[1]) and a[2] == b[2] >= 1
    assert all(torch.equal(x, y) for x, y in zip(a[0], b[0]))
    init = [p.detach().clone() for p in make_policy().trainable_params()]
    a, b = run_ranks(2, lambda comm: body(comm, both=True), timeout=60)
    assert a[2] == b[2] == 0 and all(g == 0 for g in a[1])
    assert all(torch.equal(x, y) for x, y in zip(a[0], init))


def test_rank0_writes_the_only_checkpoint_and_dp_resume_is_bit_exact(tmp_path):
    binding = CheckpointBinding("a" * 64, "b" * 64, "lora:test")

    def launch(root, steps, resume):
        def body(comm):
            if not resume and comm.rank == 0:
                RunDir.create(root, "r")
            comm.barrier()
            rd = RunDir.open(os.path.join(root, "r"))
            tr = Trainer(make_policy(), ListTok(), FnReward(varied), samples(),
                         cfg(steps=steps, prompts_per_item=1, checkpoint_every=1), comm=comm, run_dir=rd, binding=binding)
            start = tr.resume_latest() if resume else 0
            tr.train(start)
            return start, [p.detach().clone() for p in tr.params]
        return run_ranks(2, body, timeout=60)
    straight = launch(str(tmp_path / "a"), 3, False)
    launch(str(tmp_path / "b"), 2, False)
    ck = sorted(c for c in os.listdir(tmp_path / "b" / "r" / "checkpoints") if c.startswith("step-"))
    assert len(ck) == 2                                                # one directory per step, written by rank 0 alone
    resumed = launch(str(tmp_path / "b"), 3, True)
    assert [s for s, _ in resumed] == [2, 2]                           # both ranks learnt rank 0's scan result
    for r in range(2):
        for p, q in zip(straight[r][1], resumed[r][1]):
            assert torch.equal(p, q)


def test_tensor_parallel_ledger_run_equals_direct_run_and_topology_mismatch_is_refused(tmp_path):
    fix = os.path.join(FIX, "tiny_qwen3")
    led = str(tmp_path / "ledger")
    binding = CheckpointBinding("a" * 64, "b" * 64, None)

    def tp_trainer(comm, **kw):
        m = load_auto_policy(fix, LoaderOpts(tp=(comm.rank, comm.world_size)))[0]
        pol = LmPolicy(m, GrpoSampler(11, 1.0), comm)
        b = CheckpointBinding(binding.frozen_policy_sha256, binding.trainer_config_sha256, pol.lora_recipe())
        return Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, checkpoint_every=1), comm=comm,
                       topology="tp", binding=b, **kw)

    def direct(comm):
        tr = tp_trainer(comm)
        tr.step(0)
        tr.step(1)
        return [p.detach().clone() for p in tr.params]

    def separated(comm):
        if comm.rank == 0:
            RunDir.create(str(tmp_path / "runs"), "r")
        comm.barrier()
        collector, learner = tp_trainer(comm), tp_trainer(comm, run_dir=RunDir.open(str(tmp_path / "runs" / "r")))
        collector.collect_window_to(led, 0)
        c0 = learner.learn_window_from(led, 0)
        collector.learn_window_from(led, 0)
        collector.collect_window_to(led, 1, c0.lineage_sha256)
        c1 = learner.learn_window_from(led, 1, c0.lineage_sha256)
        return [p.detach().clone() for p in learner.params], (c1.tensor_parallel_world_size, c1.world_size, c1.lineage_sha256)
    want = run_ranks(2, direct, timeout=120)
    got = run_ranks(2, separated, timeout=120)
    assert got[0][1] == got[1][1] and got[0][1][:2] == (2, 1)
    for r in range(2):
        for p, q in zip(want[r], got[r][0]):
            assert torch.equal(p, q)
    # the continuation checkpoint was written for a tensor-parallel world of two: a data-parallel
    # resume of it is refused before anything is touched
    from ferrl_b200.checkpoint import (CheckpointMismatch, latest_checkpoint, latest_rollout_ledger_continuation,
                                       prepare_checkpoint)
    assert latest_checkpoint(str(tmp_path / "runs" / "r" / "checkpoints")) is None
    step, path, _ = latest_rollout_ledger_continuation(str(tmp_path / "runs" / "r" / "checkpoints"))
    assert step == 2
    with pytest.raises(CheckpointMismatch, match="topology"):
        prepare_checkpoint(path, None, world_size=2, topology="dp")
    with pytest.raises(CheckpointMismatch, match="world size"):
        prepare_checkpoint(path, None, world_size=4, topology="tp")
    assert prepare_checkpoint(path, None, world_size=2, topology="tp").manifest.rollout_ledger_continuation["kind"] == "rollout_ledger"
