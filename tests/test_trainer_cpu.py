"""Trainer behaviour on CPU: learning on a toy task, bit-exact resume, data-parallel equivalence
and lockstep failure handling with thread ranks (no GPU, no cluster)."""
import os
import threading

import pytest
import torch

from ferrl_b200.checkpoint import CheckpointBinding
from ferrl_b200.comm import PeerFailure, SoloComm, ThreadComm, run_ranks
from ferrl_b200.config import ConfigError, TrainerConfig
from ferrl_b200.lm_policy import LmPolicy
from ferrl_b200.models import DenseGradModel, DenseLoraTargets, DenseSpec, LoraSpec
from ferrl_b200.rewards import FnReward, Sample
from ferrl_b200.sampler import GrpoSampler
from ferrl_b200.telemetry import RunDir
from ferrl_b200.trainer import GradCoverageError, RunStop, Trainer

VOCAB = 32


class ListTok:
    """Tokens are space separated integers."""

    def encode(self, text):
        return [int(t) for t in text.split()]

    def decode(self, ids):
        return " ".join(str(int(i)) for i in ids)


def make_policy(seed=0, lr_rank=4):
    spec = DenseSpec(VOCAB, 32, 2, 4, 2, 8, 64, max_position_embeddings=64)
    m = DenseGradModel(spec, LoraSpec(lr_rank, 2.0 * lr_rank, DenseLoraTargets.industrial()))
    m.init_random(seed, 0.4)
    return LmPolicy(m, GrpoSampler(11, 1.0))


def echo_reward(sample, completion):
    """Reward the fraction of completion tokens equal to the prompt's last token."""
    want = sample.target
    toks = completion.split()
    return sum(1.0 for t in toks if t == want) / max(len(toks), 1)


def samples(n=8):
    return [Sample(f"{(3 * i) % VOCAB} {(5 * i + 1) % VOCAB} {7}", "7") for i in range(n)]


def cfg(**kw):
    base = dict(steps=4, group_size=6, max_new_tokens=6, lr=5e-3, beta=0.0, prompts_per_item=2, truncation_masking=False)
    base.update(kw)
    return TrainerConfig(**base)


def test_toy_task_reward_improves():
    torch.manual_seed(0)
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=30, lr=2e-2))
    assert tr.train() is RunStop.COMPLETED
    first = sum(m.reward_mean for m in tr.history[:5]) / 5
    last = sum(m.reward_mean for m in tr.history[-5:]) / 5
    assert last > first + 0.05, (first, last)
    assert all(m.grad_norm >= 0 for m in tr.history)


def test_degenerate_groups_skip_update():
    pol = make_policy()
    before = [p.detach().clone() for p in pol.trainable_params()]
    tr = Trainer(pol, ListTok(), FnReward(lambda s, c: 1.0), samples(), cfg(steps=2))
    tr.train()
    assert all(m.live_groups == 0 and m.grad_norm == 0 for m in tr.history)
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, pol.trainable_params()))
    assert tr.opt.step_t == 0


def _binding():
    return CheckpointBinding("a" * 64, "b" * 64, "lora:test")


def test_resume_is_bit_exact(tmp_path):
    def run(total, root, resume=False):
        pol = make_policy()
        rd = RunDir(str(root), "r") if resume else RunDir.create(str(root), "r")
        if resume:
            rd = RunDir.open(os.path.join(str(root), "r"))
        tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=total, checkpoint_every=2, beta=0.02),
                     run_dir=rd, binding=_binding())
        start = tr.resume_latest() if resume else 0
        tr.train(start)
        return [p.detach().clone() for p in pol.trainable_params()], tr
    straight, _ = run(4, tmp_path / "a")
    part, _ = run(2, tmp_path / "b")
    # a trainer configured for 4 steps resumes the 2-step run: steps 2..3 continue bit-exactly
    pol = make_policy()
    rd = RunDir.open(str(tmp_path / "b" / "r"))
    tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=4, checkpoint_every=2, beta=0.02),
                 run_dir=rd, binding=CheckpointBinding("a" * 64, cfg(steps=2, checkpoint_every=2, beta=0.02).digest()[:0] + "b" * 64, "lora:test"))
    assert tr.resume_latest() == 2
    tr.train(2)
    for a, b in zip(straight, pol.trainable_params()):
        assert torch.equal(a, b.detach())


def test_resume_rejects_foreign_binding(tmp_path):
    from ferrl_b200.checkpoint import CheckpointMismatch
    pol = make_policy()
    rd = RunDir.create(str(tmp_path), "r")
    tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, checkpoint_every=1), run_dir=rd,
                 binding=_binding())
    tr.train()
    pol2 = make_policy(seed=5)
    before = [p.detach().clone() for p in pol2.trainable_params()]
    tr2 = Trainer(pol2, ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, checkpoint_every=1), run_dir=rd,
                  binding=CheckpointBinding("c" * 64, "b" * 64, "lora:test"))
    with pytest.raises(CheckpointMismatch):
        tr2.resume_latest()
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, pol2.trainable_params()))   # nothing mutated


def test_world1_threadcomm_equals_solo_and_issues_no_tensor_collectives():
    a = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2))
    a.train()
    comms = ThreadComm.world(1)
    b = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2), comm=comms[0])
    b.train()
    for p, q in zip(a.params, b.params):
        assert torch.equal(p.detach(), q.detach())
    assert comms[0].collective_calls == 0


def test_dp_world2_ranks_stay_in_lockstep_and_match_single_rank_within_reassociation():
    """World 2 with one prompt per rank == world 1 with grad_accum 2 over the same prompts."""
    single = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, grad_accum_steps=2, prompts_per_item=1))
    single.train()

    def body(comm):
        tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, prompts_per_item=1), comm=comm)
        tr.train()
        return [p.detach().clone() for p in tr.params], [m.reward_mean for m in tr.history]
    res = run_ranks(2, body)
    for p0, p1 in zip(res[0][0], res[1][0]):
        assert torch.equal(p0, p1)                                   # bitwise lockstep
    for p, q in zip(single.params, res[0][0]):
        assert torch.allclose(p.detach(), q, atol=2e-5), (p.detach() - q).abs().max()


def test_dp_asymmetric_failure_rolls_back_every_rank_without_timeout():
    def body(comm):
        pol = make_policy()
        tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, prompts_per_item=1), comm=comm)
        tr.step(0)
        snap = [p.detach().clone() for p in tr.params]
        if comm.rank == 1:
            def boom(point):
                if point == "before_backward":
                    raise RuntimeError("injected backward failure")
            tr.fault_hook = boom
        with pytest.raises(PeerFailure):
            tr.step(1)
        assert all(torch.equal(a, b.detach()) for a, b in zip(snap, tr.params))
        tr.fault_hook = None
        tr.step(1)                                                   # the world is still usable
        return [p.detach().clone() for p in tr.params]
    import time
    t0 = time.time()
    res = run_ranks(2, body, timeout=30.0)
    assert time.time() - t0 < 25
    for a, b in zip(*res):
        assert torch.equal(a, b)


def test_dp_rollout_failure_is_reported_at_the_window_exchange_and_a_healthy_step_has_one_rendezvous():
    """Rollout and scoring have no rendezvous of their own under plain data parallelism: a failure there
    reaches every rank through the window-size exchange, and a healthy step enters exactly one status
    rendezvous (after backward)."""
    def body(comm):
        pol = make_policy()
        tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=3, prompts_per_item=1), comm=comm)
        coordinated = []
        orig = comm.coordinate
        comm.coordinate = lambda fn, what="": (coordinated.append(what), orig(fn, what))[1]
        tr.step(0)
        snap = [p.detach().clone() for p in tr.params]
        if comm.rank == 1:
            def boom(point):
                if point == "before_generate":
                    raise RuntimeError("injected rollout failure")
            tr.fault_hook = boom
        with pytest.raises(PeerFailure) as ei:
            tr.step(1)
        assert (ei.value.local is not None) == (comm.rank == 1)
        assert all(torch.equal(a, b.detach()) for a, b in zip(snap, tr.params))
        tr.fault_hook = None
        del coordinated[:]
        m = tr.step(1)
        assert m.live_groups > 0
        return list(coordinated), [p.detach().clone() for p in tr.params]
    res = run_ranks(2, body, timeout=30.0)
    assert res[0][0] == ["backward"] and res[1][0] == ["backward"]
    for a, b in zip(res[0][1], res[1][1]):
        assert torch.equal(a, b)


def test_uncovered_gradient_aborts():
    pol = make_policy()
    varied = FnReward(lambda s, c: float(sum(int(t) for t in c.split()) % 3))
    tr = Trainer(pol, ListTok(), varied, samples(), cfg(steps=1))
    extra = torch.nn.Parameter(torch.zeros(3))
    tr.params.append(extra)
    tr.opt.params.append(extra)
    tr.opt.m.append(torch.zeros(3))
    tr.opt.v.append(torch.zeros(3))
    with pytest.raises(GradCoverageError):
        tr.step(0)


def test_dp_one_rank_drops_a_gradient_and_every_rank_raises_coverage_error():
    """A rank whose backward left one trainable tensor without a gradient still enters the same
    tensor all-reduce as its peers (the slot is zero-filled) and the failure surfaces as a
    GradCoverageError on every rank, not as mismatched collectives (reference trainer.rs
    materialize_zero_grad_slots + reduce_accumulated_grads)."""
    varied = FnReward(lambda s, c: float(sum(int(t) for t in c.split()) % 3))

    def body(comm):
        pol = make_policy()
        tr = Trainer(pol, ListTok(), varied, samples(), cfg(steps=1, prompts_per_item=1), comm=comm)
        if comm.rank == 1:
            real = pol.backward

            def lossy(loss):
                real(loss)
                tr.params[0].grad = None
            pol.backward = lossy
        with pytest.raises(GradCoverageError):
            tr.step(0)
        return comm.collective_calls
    import time
    t0 = time.time()
    calls = run_ranks(2, body, timeout=30.0)
    assert time.time() - t0 < 25
    assert calls[0] == calls[1]          # both ranks issued the same sequence of collectives


def test_preemption_checkpoints_and_stops(tmp_path):
    rd = RunDir.create(str(tmp_path), "r")
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=10), run_dir=rd, binding=_binding())
    tr.on_step_end = lambda step, m: tr.preempt_flag.set() if step == 1 else None
    assert tr.train() is RunStop.PREEMPTED
    assert len(tr.history) == 2
    assert os.path.isdir(os.path.join(rd.checkpoints_dir, "step-2"))


def test_mu2_and_tis_and_sequence_level_run():
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(),
                 cfg(steps=2, mu=2, tis=True, beta=0.02, loss_type="grpo", top_p=0.9))
    tr.train()
    assert tr.history[-1].rollout_capture_tokens > 0 and tr.history[-1].rollout_ratio_mean > 0
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(),
                 cfg(steps=2, importance_sampling_level="sequence", loss_type="dr_grpo", clip_eps=0.01))
    tr.train()
    with pytest.raises(ConfigError):
        cfg(tis=True, importance_sampling_level="sequence").validate()


def test_ledger_collect_then_learn_equals_direct(tmp_path):
    from ferrl_b200 import ledger as L
    direct = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    direct.step(0)
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    ident = L.LedgerIdentity("a" * 64, "b" * 64, "c" * 64, "d" * 64, "e" * 64, 0, 0)
    w = L.RolloutLedgerWriter(str(tmp_path / "ledger"), ident)
    tr.collect_to_ledger(0, w)
    rec = L.RolloutLedgerReader(str(tmp_path / "ledger"), ident).read_step(0)
    learner = Trainer(make_policy(), ListTok(), FnReward(lambda s, c: 0.0), samples(), cfg(steps=1))
    learner.train_from_ledger(rec)
    for p, q in zip(direct.params, learner.params):
        assert torch.equal(p.detach(), q.detach())
    with pytest.raises(L.LedgerError):
        L.RolloutLedgerReader(str(tmp_path / "ledger"),
                              L.LedgerIdentity("f" * 64, "b" * 64, "c" * 64, "d" * 64, "e" * 64, 0, 0)).read_step(0)


_GLOO_DP_WORKER = r"""
import hashlib, os, sys
sys.path.insert(0, sys.argv[1]); sys.path.insert(0, os.path.join(sys.argv[1], "tests"))
import torch
import test_trainer_cpu as T
from ferrl_b200.comm import TorchDistComm
from ferrl_b200.rewards import FnReward
from ferrl_b200.trainer import Trainer

comm = TorchDistComm.bootstrap(backend="gloo", timeout_s=120.0)
tr = Trainer(T.make_policy(), T.ListTok(), FnReward(T.echo_reward), T.samples(),
             T.cfg(steps=2, prompts_per_item=1), comm=comm)
tr.train()
digest = hashlib.sha256(b"".join(p.detach().numpy().tobytes() for p in tr.params)).digest()
comm.require_consensus(digest, "adapters after two steps")
assert any(m.grad_norm > 0 for m in tr.history), [m.grad_norm for m in tr.history]
if comm.rank == 0:
    torch.save([p.detach().clone() for p in tr.params], sys.argv[2])
comm.barrier()
"""


def test_dp_two_gloo_processes_match_single_rank(tmp_path):
    """The same equivalence with real processes: two gloo ranks under the launcher end in
    consensus on non-trivial gradients and match the one-rank run with two accumulation steps."""
    import subprocess
    import sys
    script = tmp_path / "worker.py"
    script.write_text(_GLOO_DP_WORKER)
    out = tmp_path / "params.pt"
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2", "--master-addr", "127.0.0.1",
           "--master-port", "29671", str(script), root, str(out)]
    r = subprocess.run(cmd, capture_output=True, text=True, timeout=600)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
    single = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, grad_accum_steps=2, prompts_per_item=1))
    single.train()
    got = torch.load(out)
    for p, q in zip(single.params, got):
        assert torch.allclose(p.detach(), q, atol=2e-5), (p.detach() - q).abs().max()


def test_ledger_two_ranks_stage_shards_rank0_commits_and_learners_match_direct(tmp_path):
    """Collector and learner separated under data parallelism: each rank stages its own shard,
    rank 0 publishes one manifest covering both, and two learners that replay their shards end
    with the same adapters as two ranks that trained directly."""
    import json
    from ferrl_b200 import ledger as L
    ident = L.LedgerIdentity("a" * 64, "b" * 64, "c" * 64, "d" * 64, "e" * 64, 0, 0)
    led = str(tmp_path / "ledger")

    def direct(comm):
        tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1, prompts_per_item=1), comm=comm)
        tr.step(0)
        return [p.detach().clone() for p in tr.params]

    def collect(comm):
        tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1, prompts_per_item=1), comm=comm)
        w = L.RolloutLedgerWriter(led, ident, rank=comm.rank, world_size=comm.world_size)
        st = tr.collect_to_ledger(0, w)
        return st.rank, [g.prompt_index for g in st.groups]

    def learn(comm):
        rec = L.RolloutLedgerReader(led, ident).read_step(0, rank=comm.rank)
        tr = Trainer(make_policy(), ListTok(), FnReward(lambda s, c: 0.0), samples(), cfg(steps=1, prompts_per_item=1), comm=comm)
        tr.train_from_ledger(rec)
        return [p.detach().clone() for p in tr.params]

    want = run_ranks(2, direct)
    shards = run_ranks(2, collect)
    assert [s[0] for s in shards] == [0, 1]
    assert set(shards[0][1]).isdisjoint(shards[1][1])               # ranks drew different prompts
    win = os.path.join(led, L.step_dir_name(0))
    assert sorted(os.listdir(led)) == [L.step_dir_name(0)]           # the hidden stage is gone
    assert sorted(os.listdir(win)) == [".ferrl-ledger-owner", "manifest.json", "rank-00000.window.json",
                                       "rank-00001.window.json"]
    man = json.load(open(os.path.join(win, "manifest.json")))
    assert man["kind"] == "distributed_rollout_ledger" and man["world_size"] == 2
    assert [e["rank"] for e in man["shards"]] == [0, 1]
    both = L.RolloutLedgerReader(led, ident).read_distributed_step(0)
    assert sum(s.window_tokens for s in both) == man["window_tokens"]
    got = run_ranks(2, learn)
    for r in range(2):
        for p, q in zip(want[r], got[r]):
            assert torch.equal(p, q)
    # a learner of the wrong rank refuses the shard
    rec1 = L.RolloutLedgerReader(led, ident).read_step(0, rank=1)
    solo = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1, prompts_per_item=1))
    with pytest.raises(Exception, match="different rank/world"):
        solo.train_from_ledger(rec1)


def test_ledger_rejects_tampering_replacement_and_malformed_steps(tmp_path):
    import dataclasses
    from ferrl_b200 import ledger as L
    ident = L.LedgerIdentity("a" * 64, "b" * 64, "c" * 64, "d" * 64, "e" * 64, 0, 0)
    led = str(tmp_path / "ledger")
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    w = L.RolloutLedgerWriter(led, ident)
    st = tr.collect_to_ledger(0, w)
    assert sorted(os.listdir(os.path.join(led, L.step_dir_name(0)))) == ["manifest.json", "window.json"]
    assert L.RolloutLedgerReader(led, ident).steps() == [0]
    with pytest.raises(L.LedgerError, match="never replaced"):
        w.write_step(st)
    with pytest.raises(L.LedgerError, match="no published window"):
        L.RolloutLedgerReader(led, ident).read_step(3)
    with pytest.raises(L.LedgerError, match="source_step"):
        L.RolloutLedgerWriter(str(tmp_path / "other"), dataclasses.replace(ident, source_step=5)).write_step(st)
    with pytest.raises(L.LedgerError, match="lowercase SHA-256"):
        L.RolloutLedgerWriter(str(tmp_path / "other"), dataclasses.replace(ident, policy_sha256="XYZ"))
    # controls of the learner must agree with the collector's (schedules excepted)
    other = dataclasses.replace(st.controls, group_size=st.controls.group_size + 1)
    with pytest.raises(L.LedgerError, match="group_size"):
        L.RolloutLedgerReader(led, ident, controls=other).read_step(0)
    sched = dataclasses.replace(st.controls, effective_lr_bits=L.f64_bits(123.0))
    assert L.RolloutLedgerReader(led, ident, controls=sched).read_step(0).step == 0
    # structural validation
    bad = L.LedgerStep.from_json(st.to_json())
    bad.groups[0].token_ids[0][0] ^= 1
    with pytest.raises(L.LedgerError, match="start with its prompt"):
        bad.validate()
    bad = L.LedgerStep.from_json(st.to_json())
    bad.groups[0].completion_lens[0] = st.controls.completion_width + 1
    with pytest.raises(L.LedgerError, match="out of range"):
        bad.validate()
    with pytest.raises(L.LedgerError, match="malformed"):
        L.LedgerStep.from_json({"step": 0})
    # a flipped byte in the shard file is caught by its recorded digest
    p = w.step_path(0, 0)
    assert p.endswith(os.path.join(L.step_dir_name(0), "window.json"))
    raw = bytearray(open(p, "rb").read())
    raw[len(raw) // 2] ^= 1
    open(p, "wb").write(bytes(raw))
    with pytest.raises(L.LedgerError, match="SHA-256"):
        L.RolloutLedgerReader(led, ident).read_step(0)
    assert L.bits_f32(L.f32_bits(-0.0)) == 0.0 and L.f32_bits(-0.0) != L.f32_bits(0.0)
    assert L.bits_f64(L.f64_bits(1e-300)) == 1e-300


def test_ledger_interrupted_publication_is_invisible_and_failed_shard_aborts_every_rank(tmp_path):
    from ferrl_b200 import ledger as L
    ident = L.LedgerIdentity("a" * 64, "b" * 64, "c" * 64, "d" * 64, "e" * 64, 0, 0)
    led = str(tmp_path / "one")

    def die(where):
        if where == "before_manifest_link":
            raise OSError("disk went away")
    tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    with pytest.raises(OSError, match="disk went away"):
        tr.collect_to_ledger(0, L.RolloutLedgerWriter(led, ident, fault_hook=die))
    assert os.listdir(led) == []                                     # no stage, no claimed directory
    assert L.RolloutLedgerReader(led, ident).steps() == []
    # a directory without its commit marker is not a window
    os.mkdir(os.path.join(led, L.step_dir_name(0)))
    open(os.path.join(led, L.step_dir_name(0), "window.json"), "w").write("{}")
    assert L.RolloutLedgerReader(led, ident).steps() == []
    with pytest.raises(L.LedgerError, match="no published window"):
        L.RolloutLedgerReader(led, ident).read_step(0)
    tr2 = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    with pytest.raises(L.LedgerError, match="without a manifest"):
        tr2.collect_to_ledger(0, L.RolloutLedgerWriter(led, ident))

    # two ranks: rank 1 cannot write its shard -> both ranks raise, nothing is published, the stage is removed
    led2 = str(tmp_path / "two")

    def body(comm):
        def hook(where):
            if where == "before_shard_write" and comm.rank == 1:
                raise OSError("quota exceeded")
        t = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1, prompts_per_item=1), comm=comm)
        w = L.RolloutLedgerWriter(led2, ident, rank=comm.rank, world_size=comm.world_size, fault_hook=hook)
        try:
            t.collect_to_ledger(0, w)
        except PeerFailure as e:
            return "local" if e.local is not None else "peer"
        return "published"
    assert run_ranks(2, body) == ["peer", "local"]
    assert os.listdir(led2) == []


def test_tensor_parallel_trainer_ranks_identical_and_match_single_rank():
    """Topology "tp": both ranks hold half of every projection, roll out the SAME prompts through the
    sharded model, and apply the same update; the result equals one-rank training up to the
    reassociation of the row-parallel sums."""
    from ferrl_b200.models.loader import LoaderOpts, load_auto_policy
    fix = os.path.join(os.path.dirname(__file__), "fixtures", "tiny_qwen3")

    def policy(tp=None, comm=None):
        m = load_auto_policy(fix, LoaderOpts(tp=tp) if tp else LoaderOpts())[0]
        return LmPolicy(m, GrpoSampler(11, 1.0), comm)
    single = Trainer(policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2))
    single.train()
    assert any(m.grad_norm > 0 for m in single.history)

    def body(comm):
        tr = Trainer(policy((comm.rank, comm.world_size), comm), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2),
                     comm=comm, topology="tp")
        tr.train()
        return [p.detach().clone() for p in tr.params], [(m.reward_mean, m.completion_len_max) for m in tr.history]
    res = run_ranks(2, body, timeout=120)
    assert res[0][1] == res[1][1] == [(m.reward_mean, m.completion_len_max) for m in single.history]
    for a, b in zip(res[0][0], res[1][0]):
        assert torch.equal(a, b)
    for p, q in zip(single.params, res[0][0]):
        assert torch.allclose(p.detach(), q, atol=2e-5)
    with pytest.raises(Exception, match="need a data-parallel launch"):
        Trainer(policy(), ListTok(), FnReward(echo_reward), samples(),
                cfg(steps=1, reward_group_scope="distributed_same_prompt", group_size=2), topology="tp")


def test_collector_learner_chain_is_bit_exact_and_refuses_stale_or_foreign_windows(tmp_path):
    """Two windows through the separated path: collect from the learner's exact state, learn, hand
    the continuation's lineage to the next collector.  The chain ends where direct training ends,
    each link verifies, and a window collected from any other state is refused before mutation."""
    from ferrl_b200 import ledger as L
    from ferrl_b200.checkpoint import latest_checkpoint, latest_rollout_ledger_continuation
    direct = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2))
    direct.step(0)
    direct.step(1)
    led = str(tmp_path / "ledger")
    rd = RunDir.create(str(tmp_path / "runs"), "chain")
    collector = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2))
    learner = Trainer(make_policy(), ListTok(), FnReward(lambda s, c: 0.0), samples(), cfg(steps=7, checkpoint_every=1),
                      run_dir=rd, binding=_binding())
    collector.binding = _binding()
    assert learner.ledger_identity(0) == collector.ledger_identity(0)          # operational fields do not enter
    collector.collect_window_to(led, 0)
    c0 = learner.learn_window_from(led, 0)
    c0.verify()
    assert c0.parent_lineage_sha256 == L.ROOT_LINEAGE and c0.completed_step == 1
    # the collector adopts the learner's post-state (here: by applying the same window), then continues the chain
    collector.learn_window_from(led, 0)
    assert collector.ledger_identity(1, c0.lineage_sha256) == c0.next_identity(learner.opt.step_t)
    collector.collect_window_to(led, 1, c0.lineage_sha256)
    c1 = learner.learn_window_from(led, 1, c0.lineage_sha256)
    c1.verify()
    assert c1.parent_lineage_sha256 == c0.lineage_sha256 and c1.consumed_ledger_sha256 != c0.consumed_ledger_sha256
    for p, q in zip(direct.params, learner.params):
        assert torch.equal(p.detach(), q.detach())
    # continuation checkpoints are discovered separately and carry the chain link
    step, path, cont = latest_rollout_ledger_continuation(rd.checkpoints_dir)
    assert step == 2 and L.LedgerContinuation.from_json(cont).lineage_sha256 == c1.lineage_sha256
    assert latest_checkpoint(rd.checkpoints_dir) is None      # ordinary discovery never picks a continuation
    tampered = L.LedgerContinuation.from_json(dict(cont, consumed_ledger_sha256="0" * 64))
    with pytest.raises(L.LedgerError, match="does not follow"):
        tampered.verify()
    # a learner in any other state must not consume window 1, nor window 0 under a foreign lineage
    stale = Trainer(make_policy(seed=3), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2))
    stale.binding = _binding()
    before = [p.detach().clone() for p in stale.params]
    with pytest.raises(L.LedgerError, match="adapter_sha256"):
        stale.learn_window_from(led, 1, c0.lineage_sha256)
    with pytest.raises(L.LedgerError, match="lineage_sha256"):
        stale.learn_window_from(led, 0, c0.lineage_sha256)
    other_cfg = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=2, clip_eps=0.3))
    other_cfg.binding = _binding()
    with pytest.raises(L.LedgerError, match="trainer_config_sha256"):
        other_cfg.learn_window_from(led, 0)
    assert all(torch.equal(a, b.detach()) for a, b in zip(before, stale.params))


def test_tensor_parallel_ranks_with_diverged_adapters_are_refused_before_the_step():
    """Under tensor parallelism the adapters are replicated; a rank whose copy has drifted is caught by
    the per-step digest comparison on every rank, before any rollout or update runs (reference
    gemma4.rs:157-274 all-reduces every adapter value for the same purpose)."""
    from ferrl_b200.comm import CommMismatch

    def body(comm):
        pol = make_policy()
        tr = Trainer(pol, ListTok(), FnReward(echo_reward), samples(), cfg(steps=1), comm=comm, topology="tp")
        tr.check_replicated_adapters()                       # identical copies pass
        if comm.rank == 1:
            with torch.no_grad():
                tr.params[0].view(-1)[0] += 1e-3
        before = [p.detach().clone() for p in tr.params]
        with pytest.raises(CommMismatch, match="replicated adapter"):
            tr.step(0)
        assert all(torch.equal(a, b.detach()) for a, b in zip(before, tr.params))
        return True
    assert run_ranks(2, body, timeout=30.0) == [True, True]


def test_failed_window_leaves_no_candidate_rows(tmp_path):
    """Candidate rows logged by a window that later fails are cut from the ledger together with the
    rollback of adapters, Adam state and sampler (reference trainer.rs:7819)."""
    from ferrl_b200.telemetry import CandidateWriter, read_candidates
    path = str(tmp_path / "candidates.jsonl")
    varied = FnReward(lambda s, c: float(sum(int(t) for t in c.split()) % 3))
    tr = Trainer(make_policy(), ListTok(), varied, samples(), cfg(steps=3, candidate_log_top_k=2),
                 candidate_writer=CandidateWriter(path))
    tr.step(0)
    kept = read_candidates(path)
    assert len(kept) == 2 and all(r.step == 0 for r in kept)

    def boom(point):
        if point == "before_optimizer":
            raise RuntimeError("injected optimizer failure")
    tr.fault_hook = boom
    with pytest.raises(RuntimeError):
        tr.step(1)
    assert [r.step for r in read_candidates(path)] == [0, 0]          # step 1's rows are gone
    tr.fault_hook = None
    tr.step(1)
    assert [r.step for r in read_candidates(path)] == [0, 0, 1, 1]


def test_host_time_blocked_in_collectives_is_reported_per_step():
    """A rank that reaches an agreement point early waits there for the slowest rank: the communicator accumulates
    that time and the trainer reports the per-step difference as the ``comm_wait`` phase."""
    import time as _time
    from ferrl_b200.comm import run_ranks

    def body(comm):
        if comm.rank == 1:
            _time.sleep(0.25)
        comm.barrier()
        first = comm.wait_s
        comm.all_reduce_scalar_sum(1.0)
        return first, comm.wait_s
    (w0, w0b), (w1, w1b) = run_ranks(2, body)
    assert w0 >= 0.2 and w1 < 0.2 and w0b >= w0 and w1b >= w1

    def train(comm):
        tr = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1), comm=comm)
        return tr.step(0).phase_ms.get("comm_wait")
    waits = run_ranks(2, train, timeout=120)
    assert all(w is not None and w >= 0.0 for w in waits)
    solo = Trainer(make_policy(), ListTok(), FnReward(echo_reward), samples(), cfg(steps=1))
    assert "comm_wait" not in solo.step(0).phase_ms          # a single rank has nothing to wait for
