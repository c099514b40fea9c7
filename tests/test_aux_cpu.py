"""CPU tests of the smaller seams: rematerialisation, build identity, evaluation, discovery SDK."""
import os
import subprocess

import pytest
import torch

FIX = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def test_remat_segment_matches_plain_autograd():
    from ferrl_b200.remat import RematTape, remat_segment
    torch.manual_seed(0)
    w1 = torch.randn(6, 6, requires_grad=True)
    w2 = torch.randn(6, 6, requires_grad=True)
    frozen = torch.randn(6, 6)
    x = torch.randn(4, 6, requires_grad=True)

    def seg(h):
        return torch.tanh(h @ w1) @ frozen + torch.sin(h @ w2)

    ref = seg(seg(x)).pow(2).sum()
    gref = torch.autograd.grad(ref, (x, w1, w2))
    calls = []

    def counted(h):
        calls.append(1)
        return seg(h)

    tape = RematTape()
    h = remat_segment(counted, tape.capture(x), (w1, w2, frozen))
    y = remat_segment(counted, tape.capture(h), (w1, w2, frozen)).pow(2).sum()
    got = torch.autograd.grad(y, (x, w1, w2))
    assert torch.allclose(y, ref)
    for a, b in zip(got, gref):
        assert torch.allclose(a, b, atol=1e-6)
    assert len(calls) == 4                      # two forwards, two replays in the backward
    assert tape.bytes_held() == 2 * 4 * 6 * 4
    with torch.no_grad():
        assert torch.equal(remat_segment(seg, x, (w1, w2)), seg(x))
    # a cotangent transform is applied to the segment's input gradient only
    y2 = remat_segment(seg, x, (w1,), cot_transform=lambda g: 2 * g).sum()
    gx, gw = torch.autograd.grad(y2, (x, w1))
    px, pw = torch.autograd.grad(seg(x).sum(), (x, w1))
    assert torch.allclose(gx, 2 * px, atol=1e-6) and torch.allclose(gw, pw, atol=1e-6)


def test_build_identity_tracks_commit_and_dirt(tmp_path, monkeypatch):
    from ferrl_b200.build_identity import BuildIdentityError, require_clean, source_identity
    monkeypatch.delenv("FERRL_B200_ALLOW_DIRTY", raising=False)
    nogit = source_identity(str(tmp_path))
    assert nogit.commit == "unknown" and nogit.dirty
    with pytest.raises(BuildIdentityError):
        require_clean(nogit)
    require_clean(nogit, allow_dirty=True)
    repo = tmp_path / "r"
    repo.mkdir()
    env = dict(os.environ, GIT_AUTHOR_NAME="t", GIT_AUTHOR_EMAIL="t@t", GIT_COMMITTER_NAME="t", GIT_COMMITTER_EMAIL="t@t")
    run = lambda *a: subprocess.run(["git", *a], cwd=repo, env=env, check=True, capture_output=True)  # noqa: E731
    run("init", "-q")
    (repo / "f.txt").write_text("a")
    run("add", "f.txt")
    run("commit", "-q", "-m", "one")
    clean = source_identity(str(repo))
    assert len(clean.commit) == 40 and not clean.dirty and clean.to_json() == {"git_commit": clean.commit, "git_dirty": False}
    require_clean(clean)
    (repo / "f.txt").write_text("b")
    dirty = source_identity(str(repo))
    assert dirty.commit == clean.commit and dirty.dirty
    with pytest.raises(BuildIdentityError):
        require_clean(dirty)
    monkeypatch.setenv("FERRL_B200_ALLOW_DIRTY", "1")
    require_clean(dirty)


def _digit_fraction(sample, completion):
    """Fraction of the completion's characters that are digits (any deterministic function will do)."""
    return sum(ch.isdigit() for ch in completion) / max(1, len(completion))


def test_discovery_sdk_runs_a_task_and_publishes_outcome_last(tmp_path):
    """The narrow entry point: a task (samples + reward) and a config in, a run directory with ranked
    candidates, a health verdict, an eval comparison and a manifest-last outcome file out."""
    import json
    from ferrl_b200.config import TrainerConfig
    from ferrl_b200.discovery import Discovery, DiscoveryConfig, DiscoveryTask
    from ferrl_b200.rewards import FnReward, Sample
    from ferrl_b200.tokenizer import SyntheticTokenizer
    samples = [Sample(f"make {i} from 1 2 3", None) for i in range(6)]
    tr = TrainerConfig(steps=2, group_size=4, max_new_tokens=5, checkpoint_every=1, eos_token_id=None,
                       truncation_masking=False)
    cfg = (DiscoveryConfig.Builder(os.path.join(FIX, "tiny_qwen3")).out_dir(str(tmp_path)).trainer(tr).lora(4, 8.0)
           .candidate_top_k(3).build())
    with pytest.raises(ValueError):
        DiscoveryConfig.Builder("x").candidate_top_k(0).build()
    task = DiscoveryTask("digits", samples[:4], FnReward(_digit_fraction), samples[4:])
    out = Discovery(task, cfg, tokenizer=SyntheticTokenizer(32, 4, 8)).run()
    assert out.stop == "completed" and out.steps_run == 2 and 1 <= len(out.best) <= 3
    assert all(a.reward >= b.reward for a, b in zip(out.best, out.best[1:]))
    assert out.eval_improvement is not None
    path = os.path.join(out.run_dir, "discovery-outcome.json")
    assert os.path.exists(path) and not os.path.exists(path + ".tmp")
    js = json.load(open(path))
    assert js["steps_run"] == 2 and js["health_verdict"] == out.health_verdict and len(js["best"]) == len(out.best)
    import ferrl_b200.orchestration as orch
    assert orch.build_task.__name__ == "build_task"          # the task hook is restored after the run


def test_evaluate_compares_base_and_adapter_and_restores_state():
    from ferrl_b200.eval import EvalError, evaluate
    from ferrl_b200.policy import GenConfig
    from ferrl_b200.rewards import Sample

    class Tok:
        def encode(self, s):
            return [ord(c) % 7 for c in s]

        def decode(self, ids):
            return "".join(str(int(i)) for i in ids)

    class FakeRollout:
        def __init__(self, rows):
            self.rows = rows

        def __len__(self):
            return len(self.rows)

        def completion(self, i):
            return self.rows[i]

    class FakePolicy:
        def __init__(self):
            self.enabled, self.state, self.calls = True, 7, []

        def sampler_state(self):
            return self.state

        def restore_sampler_state(self, s):
            self.state = s

        def adapter_enabled(self):
            return self.enabled

        def set_adapter_enabled(self, on):
            self.enabled = on

        def generate_batch(self, prompts, gen, bases):
            self.state += 1
            self.calls.append((self.enabled, tuple(bases)))
            tok = 9 if self.enabled else 0          # the "adapter" emits the digit the reward likes
            return [FakeRollout([[tok] * 3 for _ in range(gen.group_size)]) for _ in prompts]

    class Nine:
        def reward_group(self, sample, comps):
            return [c.count("9") / len(c) for c in comps]

    pol = FakePolicy()
    pol.enabled = False
    samples = [Sample(f"p{i}", None) for i in range(5)]
    rep = evaluate(pol, Nine(), Tok(), samples, GenConfig(group_size=2, max_new_tokens=3), batch_prompts=2)
    assert rep.base_reward_mean == 0.0 and rep.adapter_reward_mean == 1.0 and rep.improvement() == 1.0 and len(rep.per_prompt) == 5
    assert rep.to_json()["improvement"] == 1.0 and rep.n_prompts == 5 and rep.group_size == 2
    # the adapter switch is restored; a successful evaluation keeps the sampler's progression (eval.rs:
    # successful_eval_keeps_generated_sampler_progression_and_restores_adapter)
    assert pol.enabled is False and pol.state == 7 + 6
    assert [c[0] for c in pol.calls] == [False] * 3 + [True] * 3           # paired: same row bases for both passes
    assert [c[1] for c in pol.calls[:3]] == [c[1] for c in pol.calls[3:]]
    with pytest.raises(EvalError):
        evaluate(pol, Nine(), Tok(), [], GenConfig(group_size=2, max_new_tokens=3))
    with pytest.raises(EvalError):
        evaluate(pol, Nine(), Tok(), samples, GenConfig(group_size=0, max_new_tokens=3))
    # contract errors of the reference's unit cases; a failed evaluation rolls the sampler back exactly
    gen = GenConfig(group_size=2, max_new_tokens=3)

    class Empty(Tok):
        def encode(self, s):
            return []

    class Rewards:
        def __init__(self, values):
            self.values = values

        def reward_group(self, sample, comps):
            return list(self.values)
    for tok, rew, msg in ((Empty(), Nine(), "prompt encoded to zero tokens"),
                          (Tok(), Rewards([1.0]), "reward_group returned 1 rewards for 2 completions"),
                          (Tok(), Rewards([1.0, float("nan")]), "non-finite reward"),
                          (Tok(), Rewards([float("inf"), float("inf")]), "non-finite reward")):
        pol.state, pol.enabled = 7, True
        with pytest.raises(EvalError, match=msg):
            evaluate(pol, rew, tok, samples, gen)
        assert pol.state == 7 and pol.enabled is True

    class Stuck(FakePolicy):
        def set_adapter_enabled(self, on):
            pass                                                            # full fine-tuning: nothing to switch off
    with pytest.raises(EvalError, match="cannot disable its adapter"):
        evaluate(Stuck(), Nine(), Tok(), samples, gen)

    class Short(FakePolicy):
        def generate_batch(self, prompts, gen, bases):
            return [FakeRollout([[9] * 3]) for _ in prompts]                # one row for a group of two
    with pytest.raises(EvalError, match="returned 1 completions for group_size 2"):
        evaluate(Short(), Nine(), Tok(), samples, gen)
    # means do not depend on the order of extreme finite rewards, and an improvement float32 cannot hold is refused
    from ferrl_b200.eval import EvalReport, validated_mean
    big = 3.4028234663852886e38
    assert validated_mean([big, 1.0, -big]) == validated_mean([1.0, -big, big]) == validated_mean([-big, big, 1.0])
    with pytest.raises(EvalError, match="outside finite f32"):
        EvalReport(1, 1, -big, big).improvement()


_EP_WORKER = r'''
import os, sys, torch
import torch.distributed as dist
from ferrl_b200.models import moe as M
from ferrl_b200.parallel import ep
dist.init_process_group("gloo", init_method="env://")
rank, world = dist.get_rank(), dist.get_world_size()
torch.manual_seed(11)                                   # every rank builds the same full problem
T, H, I, E, k = 37, 16, 24, 8, 2
x = torch.randn(T, H)
router = torch.randn(E, H)
gate_up = torch.randn(E, 2 * I, H) * 0.2
down = torch.randn(E, H, I) * 0.2
x_local = x[rank::world].clone().requires_grad_(True)    # each rank routes its own tokens
El = E // world

def a2a(rows, per_rank, expert_counts):
    send = [int(v) for v in per_rank.tolist()]
    recv_n = torch.zeros(world, dtype=torch.long)
    dist.all_to_all_single(recv_n, torch.tensor(send, dtype=torch.long))
    recv = rows.new_empty((int(recv_n.sum()), rows.shape[1]))
    dist.all_to_all_single(recv, rows.contiguous(), [int(v) for v in recv_n.tolist()], send)
    rec = None
    if expert_counts is not None:
        rec = torch.zeros(world, El, dtype=torch.long)
        dist.all_to_all_single(rec, expert_counts.contiguous().long())
    return recv, recv_n, rec

ep.install(ep.EpContext(rank, world, all_to_all_rows=a2a))
y = ep.sparse_moe(x_local, router, gate_up[rank * El:(rank + 1) * El], down[rank * El:(rank + 1) * El], k, None, None)
ep.install(None)
ref = M.sparse_moe_block(x[rank::world], router, gate_up, down, k)
err = (y - ref).abs().max().item()
assert err < 1e-4, err
print("EP_OK", rank, err, flush=True)
dist.destroy_process_group()
'''


def test_expert_parallel_host_path_two_gloo_ranks():
    """Experts sharded over two CPU ranks (dispatch and combine through gloo all-to-all) give the same
    block output as one rank holding every expert."""
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", MASTER_ADDR="127.0.0.1", MASTER_PORT="29647", PYTHONPATH=root)
        procs.append(subprocess.Popen([sys.executable, "-c", _EP_WORKER], env=env, stdout=subprocess.PIPE,
                                      stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=240)
        assert p.returncode == 0 and "EP_OK" in out, err[-2500:]


def test_examples_run_end_to_end_on_cpu(tmp_path):
    """Every CPU example runs as a user would start it; the run report reads what the trainer wrote."""
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

    def run(*args):
        r = subprocess.run([sys.executable, *args], cwd=root, capture_output=True, text=True, timeout=600)
        assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-4000:]
        return r.stdout

    out = run("examples/countdown_grpo.py", "--steps", "2", "--out", str(tmp_path))
    assert "COMPLETED" in out
    runs = [d for d in os.listdir(tmp_path) if os.path.isdir(tmp_path / d)]
    assert len(runs) == 1
    report = run("examples/runreport.py", str(tmp_path / runs[0]))
    assert "2 steps" in report
    assert "reward per step" in run("examples/minimal_task.py")
    assert "step 0" in run("examples/countdown_grpo_qwen35.py", "--steps", "1", "--moe")
    # two gloo ranks as one tensor-parallel group, replicated and sequence-sharded residual stream: the same
    # adapters come out of both layouts (the collectives sum in rank order either way)
    digests = []
    for port, extra in ((29821, ()), (29822, ("--sequence-parallel",))):
        out = run("-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
                  "--master-port", str(port), "examples/gemma_tensor_parallel.py", "--steps", "2", "--out",
                  str(tmp_path / f"tp{port}"), *extra)
        line = [l for l in out.splitlines() if "all ranks hold identical adapters" in l]
        assert line and "step 1" in out, out[-1500:]
        digests.append(line[0].split()[-1])
    assert digests[0] == digests[1]


def _discovery_setup(tmp_path, verify, **task_kw):
    from ferrl_b200.config import TrainerConfig
    from ferrl_b200 import discovery as D
    from ferrl_b200.rewards import FnReward, Sample
    samples = [Sample(f"make {i} from 1 2 3", None) for i in range(6)]
    tr = TrainerConfig(steps=2, group_size=4, max_new_tokens=5, checkpoint_every=1, eos_token_id=None,
                       truncation_masking=False)
    contract = D.MetricContract("digit share", "fraction", D.HIGHER_IS_BETTER, 0.25, 0.05)
    task = D.DiscoveryTask("digits", samples[:4], FnReward(_digit_fraction), samples[4:], version=2,
                           metric_contract=contract, verify_candidate=verify, **task_kw)
    b = (D.DiscoveryConfig.Builder(os.path.join(FIX, "tiny_qwen3")).out_dir(str(tmp_path / "runs")).trainer(tr)
         .lora(4, 8.0).candidate_top_k(4).artifact_output(str(tmp_path / "bundle")))
    return D, task, contract, b


def test_discovery_verified_outcome_publishes_bundle_manifest_last(tmp_path):
    import json
    from ferrl_b200.tokenizer import SyntheticTokenizer
    seen = []

    def verify(cand):
        seen.append(cand)
        score = 0.25 + 0.1 * (len(seen) == 2) + 0.2 * (len(seen) == 3)      # third candidate is strongest
        if len(seen) == 1:
            return D.CandidateVerification.rejected("does not parse")
        return D.CandidateVerification.measured(D.FinalEvidence(True, D.MetricReport.of(contract, score),
                                                                {"program": cand.completion}, {"trials": 3}))
    D, task, contract, b = _discovery_setup(tmp_path, verify)
    out = D.Discovery(task, b.build(), tokenizer=SyntheticTokenizer(32, 4, 8)).run()
    assert out.kind == "verified" and out.artifact is not None and len(seen) >= 3
    assert all(len(c.provenance_sha256) == 64 for c in seen)
    assert [c.search_reward for c in seen] == sorted((c.search_reward for c in seen), reverse=True)
    art = out.artifact
    assert sorted(os.listdir(art.output)) == sorted(D.ARTIFACT_FILES + (D.ARTIFACT_MANIFEST_FILE,))
    man = D.verify_artifact_bundle(art.output)
    assert man["contract"] == "ferrl.discovery-artifact.v1" and man["task"] == {"name": "digits", "version": 2}
    assert man["candidate_sha256"] == seen[2].provenance_sha256 and abs(art.metric.candidate - 0.45) < 1e-12
    assert json.load(open(art.payload_path)) == {"program": seen[2].completion}
    ev = json.load(open(art.verification_evidence_path))
    assert ev["held_out_correct"] is True and ev["evidence"] == {"trials": 3}
    assert json.load(open(os.path.join(art.output, "launch.json")))["launch_sha256"] == man["launch_sha256"]
    assert json.load(open(os.path.join(out.run_dir, "discovery-outcome.json")))["kind"] == "verified"
    # a tampered file is caught; a second run refuses to overwrite the bundle before loading anything
    with open(art.payload_path, "a") as f:
        f.write(" ")
    with pytest.raises(D.DiscoveryError, match="does not match the manifest"):
        D.verify_artifact_bundle(art.output)
    with pytest.raises(D.InvalidConfiguration, match="already exists"):
        D.Discovery(task, b.build(), tokenizer=SyntheticTokenizer(32, 4, 8)).run()


def test_discovery_no_win_reasons_preemption_and_validation(tmp_path):
    import threading
    from ferrl_b200.tokenizer import SyntheticTokenizer
    D, task, contract, b = _discovery_setup(tmp_path, None)
    tok = SyntheticTokenizer(32, 4, 8)

    def outcome(verify, sub):
        t = D.DiscoveryTask(task.name, task.samples, task.reward_fn, task.eval_samples, 2, contract, verify)
        cfg = b.out_dir(str(tmp_path / sub)).artifact_output(str(tmp_path / (sub + "-bundle"))).build()
        return D.Discovery(t, cfg, tokenizer=tok).run(), str(tmp_path / (sub + "-bundle"))

    out, bundle = outcome(lambda c: D.CandidateVerification.rejected(" "), "rej")
    assert out.kind == "no_win" and out.no_win.reason == D.NO_WIN_CANDIDATES_REJECTED
    assert out.no_win.detail == "candidate rejected without task detail" and not os.path.exists(bundle)
    out, _ = outcome(lambda c: D.CandidateVerification.measured(
        D.FinalEvidence(False, D.MetricReport.of(contract, 0.9), {}, {})), "wrong")
    assert out.no_win.reason == D.NO_WIN_HELD_OUT_INCORRECT
    # exactly at the margin is not a win: the improvement must strictly exceed it
    out, _ = outcome(lambda c: D.CandidateVerification.measured(
        D.FinalEvidence(True, D.MetricReport.of(contract, 0.25 + 0.05), {}, {})), "margin")
    assert out.no_win.reason == D.NO_WIN_NO_MATERIAL_METRIC_WIN and out.no_win.candidates_checked >= 1
    # evidence measured under another contract is an error, and so is a crashing verifier
    other = D.MetricContract("digit share", "fraction", D.HIGHER_IS_BETTER, 0.0, 0.05)
    with pytest.raises(D.InvalidFinalEvidence, match="launch-frozen"):
        outcome(lambda c: D.CandidateVerification.measured(D.FinalEvidence(True, D.MetricReport.of(other, 1.0), {}, {})), "c2")
    with pytest.raises(D.TaskVerificationError, match="sandbox died"):
        outcome(lambda c: (_ for _ in ()).throw(RuntimeError("sandbox died")), "crash")
    # cooperative preemption: stops after the step in flight, checkpoints, verifies nothing
    flag = threading.Event()
    flag.set()
    called = []
    t = D.DiscoveryTask(task.name, task.samples, task.reward_fn, task.eval_samples, 2, contract,
                        lambda c: called.append(c))
    cfg = b.out_dir(str(tmp_path / "pre")).artifact_output(str(tmp_path / "pre-bundle")).preemption_flag(flag).build()
    out = D.Discovery(t, cfg, tokenizer=tok).run()
    assert out.kind == "preempted" and out.steps_run == 1 and not called and not os.path.exists(cfg.artifact_output)
    assert os.path.isdir(os.path.join(out.run_dir, "checkpoints"))
    # validation before anything is loaded
    with pytest.raises(D.InvalidConfiguration, match="contain"):
        b.out_dir(str(tmp_path / "a" / "runs")).artifact_output(str(tmp_path / "a")).build()
    with pytest.raises(D.InvalidConfiguration, match="task name"):
        D.TaskIdentity("Has Space")
    with pytest.raises(D.InvalidFinalEvidence):
        D.MetricContract(" padded", "s", D.LOWER_IS_BETTER, 1.0, 0.0).validate()
    with pytest.raises(D.InvalidFinalEvidence):
        D.MetricContract("t", "s", D.LOWER_IS_BETTER, 1.0, -0.1).validate()
    low = D.MetricContract("latency", "us", D.LOWER_IS_BETTER, 100.0, 2.0)
    assert D.MetricReport.of(low, 97.0).is_material_win() and not D.MetricReport.of(low, 98.0).is_material_win()
    assert D.metric_is_stronger(D.MetricReport.of(low, 90.0), D.MetricReport.of(low, 95.0))


def test_discovery_bundle_publication_failure_leaves_nothing(tmp_path):
    from ferrl_b200 import discovery as D
    from ferrl_b200.telemetry import CandidateRecord
    rec = CandidateRecord(1, 0, 1, 3, 2, 0.5, 4, "1 2 3 4")
    contract = D.MetricContract("m", "u", D.HIGHER_IS_BETTER, 0.0, 0.0)
    ev = D.FinalEvidence(True, D.MetricReport.of(contract, 1.0), {"x": 1}, {})

    def die(where):
        raise OSError("no space left")
    out = str(tmp_path / "bundle")
    with pytest.raises(OSError):
        D.publish_verified_artifact(out, D.TaskIdentity("t"), "run", b'{"launch_sha256": "ab"}', b"{}", rec, ev, fault_hook=die)
    assert os.listdir(tmp_path) == []
    art = D.publish_verified_artifact(out, D.TaskIdentity("t"), "run", b'{"launch_sha256": "ab"}', b"{}", rec, ev)
    assert D.verify_artifact_bundle(art.output)["candidate_sha256"] == rec.digest()
    with pytest.raises(D.InvalidConfiguration, match="already exists"):
        D.publish_verified_artifact(out, D.TaskIdentity("t"), "run", b"{}", b"{}", rec, ev)


@pytest.mark.parametrize("world,softcap,temperature", [(2, 0.0, 1.0), (4, 30.0, 0.7)])
def test_vocabulary_sharded_logprob_head_equals_the_full_head_on_thread_ranks(world, softcap, temperature):
    """Each tensor-parallel rank scores 1 / world of the vocabulary; values and hidden-state gradients must equal
    the unsharded log-softmax gather, identically on every rank."""
    import torch
    from ferrl_b200.comm import run_ranks
    from ferrl_b200.ops import eager
    from ferrl_b200.parallel.tp import sharded_logprob_gather
    g = torch.Generator().manual_seed(3)
    N, H, V = 37, 24, 64 * world
    h0 = torch.randn(N, H, generator=g)
    w = torch.randn(V, H, generator=g) * 0.5
    t = torch.randint(0, V, (N,), generator=g)
    dlp = torch.randn(N, generator=g)
    hr = h0.clone().requires_grad_()
    ref = eager.logprob_gather(hr, w, t, temperature, softcap)
    ref.backward(dlp)

    def body(comm):
        h = h0.clone().requires_grad_()
        lp = sharded_logprob_gather(h, w, t, temperature, softcap, comm)
        assert lp is not None
        lp.backward(dlp)
        return lp.detach(), h.grad
    outs = run_ranks(world, body, timeout=60)
    for lp, grad in outs:
        assert torch.allclose(lp, ref.detach(), atol=2e-5, rtol=1e-5)
        assert torch.allclose(grad, hr.grad, atol=2e-5, rtol=1e-4)
        assert torch.equal(lp, outs[0][0]) and torch.equal(grad, outs[0][1])      # every rank holds the same bits
    assert sharded_logprob_gather(h0, w[:V - 1], t.clamp(max=V - 2), 1.0, 0.0, type("C", (), {"world_size": world, "rank": 0})()) is None
