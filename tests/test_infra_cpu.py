"""Host-side infrastructure: communicators, config, checkpoints, telemetry, rewards, sandbox,
artifact audit, orchestration and CLI."""
import json
import os
import sys
import threading
import time

import pytest
import torch

from ferrl_b200 import checkpoint as CK, telemetry as T
from ferrl_b200.comm import (CommMismatch, CommPoisoned, CommTimeout, NcclConfig, CommConfigError, PeerFailure, SoloComm,
                             ThreadComm, run_ranks)
from ferrl_b200.config import ConfigError, RunConfig, ScalarSchedule, TrainerConfig
from ferrl_b200.optim import AdamWParams, FerrlAdamW, OptimizerState

FIX = os.path.join(os.path.dirname(__file__), "fixtures")


# ------------------------------------------------------------------ comm
def test_threadcomm_sums_in_rank_order_and_gathers():
    def body(c):
        t = [torch.full((3,), float(c.rank + 1))]
        c.all_reduce_sum(t)
        return t[0].tolist(), c.all_reduce_scalar_sum(c.rank + 1), c.all_gather_bytes(bytes([c.rank])), \
            c.all_reduce_scalars_sum([1.0, c.rank])
    for vals, s, g, packed in run_ranks(4, body):
        assert vals == [10.0] * 3 and s == 10.0 and g == [b"\x00", b"\x01", b"\x02", b"\x03"] and packed == [4.0, 6.0]


def test_threadcomm_mismatch_timeout_poison_and_consensus():
    def mism(c):
        c.all_reduce_sum([torch.zeros(2 + c.rank)])
    with pytest.raises(CommMismatch):
        run_ranks(2, mism)

    def lonely(c):
        if c.rank == 0:
            c.all_reduce_scalar_sum(1.0)
    with pytest.raises(CommTimeout):
        run_ranks(2, lonely, timeout=0.3)

    def cons(c):
        c.require_consensus(b"same", "x")
        with pytest.raises(CommMismatch):
            c.require_consensus(bytes([c.rank]), "y")
        return True
    assert run_ranks(3, cons) == [True] * 3
    comms = ThreadComm.world(2)
    comms[0].poison("dead")
    with pytest.raises(CommPoisoned):
        comms[1].all_reduce_scalar_sum(0.0)
    with pytest.raises(CommMismatch):
        SoloComm().validate_all_reduce_sum([torch.zeros(2, dtype=torch.bfloat16)])


def test_coordinate_turns_one_failure_into_a_failure_everywhere():
    def body(c):
        def f():
            if c.rank == 2:
                raise ValueError("boom")
            return c.rank
        try:
            c.coordinate(f, "stage")
        except PeerFailure as e:
            return ("failed", e.local is not None)
        return ("ok", False)
    assert run_ranks(3, body) == [("failed", False), ("failed", False), ("failed", True)]


def test_nccl_config_from_env():
    assert NcclConfig.from_env({}) is None
    c = NcclConfig.from_env({"RANK": "1", "WORLD_SIZE": "4", "LOCAL_RANK": "1", "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": "1234"})
    assert (c.rank, c.world_size, c.init_method) == (1, 4, "tcp://127.0.0.1:1234")
    c = NcclConfig.from_env({"FERRL_NCCL_RENDEZVOUS": "/tmp/rdv", "SLURM_PROCID": "0", "SLURM_NTASKS": "2", "SLURM_LOCALID": "0"})
    assert c.init_method == "file:///tmp/rdv"
    with pytest.raises(CommConfigError):
        NcclConfig.from_env({"RANK": "5", "WORLD_SIZE": "4"})
    with pytest.raises(CommConfigError):
        NcclConfig.from_env({"FERRL_NCCL_RENDEZVOUS": "/tmp/x", "SLURM_PROCID": "zero", "SLURM_NTASKS": "2", "SLURM_LOCALID": "0"})


def test_gloo_process_group_two_ranks(tmp_path):
    """The torch.distributed communicator on CPU (gloo), as two real processes."""
    import subprocess
    import sys
    code = ("import torch, os; from ferrl_b200.comm import TorchDistComm; c = TorchDistComm.bootstrap(backend='gloo', timeout_s=60);"
            "t=[torch.full((4,), float(c.rank+1))]; c.all_reduce_sum(t); assert t[0].tolist()==[3.0]*4;"
            "assert c.all_reduce_scalar_sum(c.rank+1)==3.0; assert c.all_gather_bytes(bytes([c.rank]))==[b'\\x00', b'\\x01'];"
            "c.require_consensus(b'x','cfg'); c.barrier(); print('GLOO_OK', c.rank)")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT="29641",
                   PYTHONPATH=root)
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    for p in procs:
        out, err = p.communicate(timeout=180)
        assert p.returncode == 0 and "GLOO_OK" in out, err[-2000:]


# ---------------------------------------------------------------- config
def test_trainer_config_validation_and_schedules():
    c = TrainerConfig()
    c.validate()
    assert (c.loss_type, c.mu, c.beta, c.max_grad_norm, c.truncation_masking) == ("dapo", 1, 0.0, 1.0, True)
    for bad in (dict(steps=0), dict(mu=0), dict(group_size=1), dict(clip_eps=1.0), dict(temperature=0.0),
                dict(lr=-1.0), dict(max_grad_norm=0.0), dict(tis_imp_ratio_cap=0.5), dict(checkpoint_every=0),
                dict(lr_schedule=ScalarSchedule.constant(1.0), warmup_steps=2)):
        with pytest.raises(ConfigError):
            TrainerConfig(**bad).validate()
    c = TrainerConfig(lr=1.0, warmup_steps=4)
    assert [c.lr_at(i) for i in range(5)] == [0.25, 0.5, 0.75, 1.0, 1.0]
    s = ScalarSchedule.linear(0.0, 1.0, 10)
    assert s.at(0) == 0.0 and s.at(5) == 0.5 and s.at(99) == 1.0
    c = TrainerConfig(steps=20, beta_schedule=ScalarSchedule([(0, 0.0), (10, 0.1)]))
    c.validate()
    assert c.requires_reference_policy() and abs(c.beta_at(5) - 0.05) < 1e-12
    assert TrainerConfig.from_json(c.to_json()).digest() == c.digest()
    with pytest.raises(ConfigError):
        TrainerConfig.from_json({"stepz": 3})


def test_run_config_strict_json_eos_modes_and_digest():
    base = {"task": "countdown", "model_dir": "/m", "trainer": {"steps": 2}}
    cfg = RunConfig.from_json(base)
    assert cfg.eos_selection == "checkpoint" and "eos_token_id" not in cfg.to_json()["trainer"]
    assert RunConfig.from_json(dict(base, trainer={"steps": 2, "eos_token_id": 7})).eos_selection == "explicit"
    d = RunConfig.from_json(dict(base, trainer={"steps": 2, "eos_token_id": "none"}))
    assert d.eos_selection == "disabled" and d.to_json()["trainer"]["eos_token_id"] == "none"
    for bad in (dict(base, trainer={"steps": 2, "eos_token_id": None}), dict(base, extra=1), dict(base, task="chess"),
                dict(base, policy={"lora_rnk": 1}),
                dict(base, distributed={"enabled": True}, tensor_parallel={"enabled": True, "rank": 0, "world_size": 2})):
        with pytest.raises(ConfigError):
            RunConfig.from_json(bad)
    a = RunConfig.from_json(dict(base, tensor_parallel={"enabled": True, "rank": 0, "world_size": 2}))
    b = RunConfig.from_json(dict(base, tensor_parallel={"enabled": True, "rank": 1, "world_size": 2}))
    assert a.digest() == b.digest() and a.digest() != cfg.digest()


# ------------------------------------------------------------ checkpoint
def _ck(tmp, step=3, adapters=None):
    adapters = adapters or [torch.randn(4, 8), torch.zeros(8, 4)]
    opt = OptimizerState(5, [torch.ones_like(a) for a in adapters], [torch.full_like(a, 2.0) for a in adapters])
    b = CK.CheckpointBinding("a" * 64, "b" * 64, "lora:r4")
    path = CK.save_checkpoint(str(tmp), step, adapters, opt, b"sampler", b, world_size=2)
    return path, adapters, b


def test_checkpoint_round_trip_and_layout(tmp_path):
    path, adapters, b = _ck(tmp_path)
    assert sorted(os.listdir(path)) == ["adapter.safetensors", "manifest.json", "optimizer.safetensors", "topology.json"]
    man = json.load(open(os.path.join(path, "manifest.json")))
    # exactly the reference manifest's field set (its decoder rejects unknown fields)
    assert sorted(man) == sorted(["format_version", "step", "num_vars", "optimizer_step_t", "optimizer_num_vars",
                                  "sampler_state", "lora_recipe", "rollout_ledger_continuation", "ordinary_checkpoint"])
    assert man["format_version"] == 4 and man["step"] == 3 and man["num_vars"] == 2 and man["optimizer_step_t"] == 5
    from safetensors.torch import load_file
    assert sorted(load_file(os.path.join(path, "adapter.safetensors"))) == ["lora.00000", "lora.00001"]
    assert sorted(load_file(os.path.join(path, "optimizer.safetensors"))) == ["m.00000", "m.00001", "v.00000", "v.00001"]
    params = [torch.nn.Parameter(torch.zeros(4, 8)), torch.nn.Parameter(torch.ones(8, 4))]
    lc = CK.load_checkpoint(path, b, params, world_size=2, topology="dp")
    assert all(torch.equal(p.detach(), a) for p, a in zip(params, adapters))
    assert lc.optimizer.step == 5 and lc.manifest.sampler_bytes() == b"sampler"
    assert CK.latest_checkpoint(str(tmp_path)) == (3, path)
    with pytest.raises(CK.CheckpointError):
        CK.save_checkpoint(str(tmp_path), 3, adapters, None, None, b)          # never replaced


def test_checkpoint_corruption_and_binding_are_rejected_before_mutation(tmp_path):
    path, adapters, b = _ck(tmp_path)
    params = [torch.nn.Parameter(torch.zeros(4, 8)), torch.nn.Parameter(torch.ones(8, 4))]
    for wrong in (CK.CheckpointBinding("c" * 64, "b" * 64, "lora:r4"), CK.CheckpointBinding("a" * 64, "d" * 64, "lora:r4"),
                  CK.CheckpointBinding("a" * 64, "b" * 64, "lora:r8")):
        with pytest.raises(CK.CheckpointMismatch):
            CK.load_checkpoint(path, wrong, params)
    with pytest.raises(CK.CheckpointMismatch):
        CK.load_checkpoint(path, b, params, world_size=4)
    with pytest.raises(CK.CheckpointMismatch):
        CK.load_checkpoint(path, b, [torch.nn.Parameter(torch.zeros(4, 9)), params[1]])
    with open(os.path.join(path, "adapter.safetensors"), "r+b") as f:
        f.seek(-1, 2)
        f.write(b"\x55")
    with pytest.raises(CK.CheckpointMismatch):
        CK.load_checkpoint(path, b, params)
    assert torch.equal(params[0].detach(), torch.zeros(4, 8))
    with pytest.raises(CK.CheckpointMismatch):
        CK.CheckpointBinding("xyz", "b" * 64)


def _ref_domain(domain, fields):
    """Independent restatement of the reference's length-prefixed, domain-separated SHA-256
    (crates/ferrl/src/checkpoint.rs:447-456)."""
    import hashlib
    import struct
    h = hashlib.sha256()
    h.update(struct.pack("<Q", len(domain)) + domain.encode())
    for f in fields:
        h.update(struct.pack("<Q", len(f)) + f)
    return h.hexdigest()


def test_checkpoint_identity_follows_the_reference_formulas(tmp_path):
    """Golden manifest: every digest of the identity block recomputed from the reference's
    formulas (domains ferrl.ordinary-checkpoint.*, step_t bound into the optimizer digest, schema
    as JSON of (recipe, [(key, dims, dtype)]), envelope as the struct's compact JSON)."""
    import struct
    path, adapters, b = _ck(tmp_path)
    man = json.load(open(os.path.join(path, "manifest.json")))
    ident = man["ordinary_checkpoint"]
    raw_a = open(os.path.join(path, "adapter.safetensors"), "rb").read()
    raw_o = open(os.path.join(path, "optimizer.safetensors"), "rb").read()
    assert ident["kind"] == "ordinary"
    assert ident["adapter_sha256"] == _ref_domain("ferrl.ordinary-checkpoint.adapter.v1", [raw_a])
    assert ident["optimizer_sha256"] == _ref_domain("ferrl.ordinary-checkpoint.optimizer.v1", [struct.pack("<Q", 5), raw_o])
    assert ident["sampler_sha256"] == _ref_domain("ferrl.ordinary-checkpoint.sampler.v1", [b"sampler"])
    schema = '["lora:r4",[["lora.00000",[4,8],"f32"],["lora.00001",[8,4],"f32"]]]'
    assert ident["tensor_schema_sha256"] == _ref_domain("ferrl.ordinary-checkpoint.tensor-schema.v1", [schema.encode()])
    env = ('{"format_version":4,"kind":"ordinary","step":3,"num_vars":2,"lora_recipe":"lora:r4","optimizer_step_t":5,'
           '"optimizer_num_vars":2,"frozen_policy_sha256":"%s","trainer_config_sha256":"%s","tensor_schema_sha256":"%s",'
           '"adapter_sha256":"%s","optimizer_sha256":"%s","sampler_sha256":"%s"}'
           % ("a" * 64, ident["trainer_config_sha256"], ident["tensor_schema_sha256"], ident["adapter_sha256"],
              ident["optimizer_sha256"], ident["sampler_sha256"]))
    assert ident["state_envelope_sha256"] == _ref_domain("ferrl.ordinary-checkpoint.state-envelope.v1", [env.encode()])
    # world size and topology live inside trainer_config_sha256, not in manifest fields
    assert ident["trainer_config_sha256"] == CK.bound_trainer_config_sha256("b" * 64, 2, "dp") != "b" * 64
    assert CK.LOCK_SUFFIX == ".writer-lock"


def test_checkpoint_tampered_counters_kind_and_optimizer_payload_are_rejected(tmp_path):
    path, adapters, b = _ck(tmp_path)
    mp = os.path.join(path, "manifest.json")
    good = json.load(open(mp))
    params = [torch.nn.Parameter(torch.zeros(4, 8)), torch.nn.Parameter(torch.ones(8, 4))]

    def rewrite(mut):
        man = json.loads(json.dumps(good))
        mut(man)
        json.dump(man, open(mp, "w"))
    for mut in (lambda m: m.__setitem__("optimizer_step_t", 6),          # wrong Adam bias correction on resume
                lambda m: m.__setitem__("optimizer_num_vars", 1),
                lambda m: m.__setitem__("num_vars", 1),
                lambda m: m.__setitem__("step", 4),
                lambda m: m["ordinary_checkpoint"].__setitem__("kind", "rollout_ledger"),
                lambda m: m.__setitem__("world_size", 2)):                # not a manifest field
        rewrite(mut)
        with pytest.raises(CK.CheckpointMismatch):
            CK.load_checkpoint(path, b, params)
        assert torch.equal(params[0].detach(), torch.zeros(4, 8))
    rewrite(lambda m: None)
    CK.load_checkpoint(path, b, params, world_size=2, topology="dp")
    # an edited topology side file no longer matches what trainer_config_sha256 binds
    json.dump({"world_size": 4, "topology": "dp"}, open(os.path.join(path, "topology.json"), "w"))
    with pytest.raises(CK.CheckpointMismatch):
        CK.load_checkpoint(path, b, params)
    json.dump({"world_size": 2, "topology": "dp"}, open(os.path.join(path, "topology.json"), "w"))
    # optimizer payload with an extra tensor / a moment of the wrong shape (digests re-sealed by an attacker
    # who cannot be told from a writer bug): refused by the key and shape checks
    from safetensors.torch import load_file, save_file
    op = os.path.join(path, "optimizer.safetensors")
    ot = load_file(op)
    for bad in ({**ot, "m.00002": torch.zeros(1)}, {**ot, "v.00001": torch.zeros(3, 3)}):
        save_file(bad, op)
        man = json.loads(json.dumps(good))
        ident = man["ordinary_checkpoint"]
        ident["optimizer_sha256"] = CK.optimizer_payload_sha256(5, open(op, "rb").read())
        ident["state_envelope_sha256"] = CK.state_envelope_sha256(4, "ordinary", 3, 2, "lora:r4", 5, 2, ident)
        json.dump(man, open(mp, "w"))
        with pytest.raises(CK.CheckpointMismatch):
            CK.load_checkpoint(path, b, params)


def test_latest_checkpoint_skips_ledger_continuations(tmp_path):
    path, adapters, b = _ck(tmp_path, step=2)
    opt = OptimizerState(5, [torch.ones_like(a) for a in adapters], [torch.full_like(a, 2.0) for a in adapters])
    CK.save_checkpoint(str(tmp_path), 7, adapters, opt, b"s", b, continuation={"kind": "rollout_ledger", "completed_step": 7})
    assert CK.latest_checkpoint(str(tmp_path)) == (2, path)
    assert CK.latest_rollout_ledger_continuation(str(tmp_path))[0] == 7


def test_failed_publication_leaves_nothing_and_newer_malformed_is_an_error(tmp_path):
    def hook(stage):
        if stage == "optimizer_written":
            raise OSError("disk full")
    b = CK.CheckpointBinding("a" * 64, "b" * 64, None)
    with pytest.raises(OSError):
        CK.save_checkpoint(str(tmp_path), 1, [torch.zeros(2)], None, None, b, fault_hook=hook)
    assert CK.latest_checkpoint(str(tmp_path)) is None and not any(n.startswith("step-1") and "staging" in n for n in os.listdir(tmp_path))
    _ck(tmp_path, step=2)
    os.makedirs(tmp_path / "step-9")
    with pytest.raises(CK.CheckpointMismatch):
        CK.latest_checkpoint(str(tmp_path))


def test_bare_adapter_round_trip(tmp_path):
    a = [torch.randn(2, 3), torch.randn(3, 2)]
    CK.save_adapter(str(tmp_path / "a.safetensors"), a, "lora:x")
    p = [torch.nn.Parameter(torch.zeros(2, 3)), torch.nn.Parameter(torch.zeros(3, 2))]
    CK.load_adapter(str(tmp_path / "a.safetensors"), p, "lora:x")
    assert all(torch.equal(x.detach(), y) for x, y in zip(p, a))
    with pytest.raises(CK.CheckpointMismatch):
        CK.load_adapter(str(tmp_path / "a.safetensors"), p, "lora:y")


def test_adamw_matches_torch_and_state_round_trips():
    torch.manual_seed(0)
    p = [torch.nn.Parameter(torch.randn(5, 3).double().float())]
    q = [torch.nn.Parameter(p[0].detach().clone())]
    ours = FerrlAdamW(p, AdamWParams(lr=1e-2, weight_decay=0.1))
    ref = torch.optim.AdamW(q, lr=1e-2, weight_decay=0.1, eps=1e-8)
    for _ in range(5):
        g = torch.randn(5, 3)
        ours.step([g])
        q[0].grad = g.clone()
        ref.step()
    assert torch.allclose(p[0], q[0], atol=1e-6)
    st = ours.state()
    other = FerrlAdamW([torch.nn.Parameter(torch.zeros(5, 3))])
    other.load_state(st)
    assert other.step_t == 5 and torch.equal(other.m[0], ours.m[0])
    with pytest.raises(ValueError):
        other.load_state(OptimizerState(1, [torch.zeros(2)], [torch.zeros(2)]))


# ------------------------------------------------------------- telemetry
def test_metrics_sanitising_candidates_and_health(tmp_path):
    rd = T.RunDir.create(str(tmp_path), "run")
    with pytest.raises(FileExistsError):
        T.RunDir.create(str(tmp_path), "run")
    w = T.MetricsWriter(rd.metrics_path)
    for i in range(6):
        w.append(T.Metrics(step=i, reward_mean=0.1 * i, grad_norm=(100.0 if i == 4 else 1.0), step_secs=1.0,
                           loss=float("nan") if i == 5 else 0.0))
    rows = T.read_metrics(rd.metrics_path)
    assert rows[5].loss == 0.0 and "loss" in rows[5].nonfinite_fields
    kinds = {a.kind for a in T.detect_anomalies(rows)}
    assert {"non_finite", "grad_spike"} <= kinds and T.detect_anomalies([])[0].kind == "telemetry_dark"
    stall = [T.Metrics(step=i, reward_mean=0.5, frac_reward_zero_std=1.0) for i in range(6)]
    assert any(a.kind == "reward_stall" for a in T.detect_anomalies(stall))
    signer = T.CandidateSigner("f" * 64)
    cw = T.CandidateWriter(rd.candidates_path, signer)
    cw.append(T.CandidateRecord(1, 0, 1, 3, 0, 0.9, 5, "answer"))
    rec = T.read_candidates(rd.candidates_path)[0]
    T.verify_candidate(rec, signer.public_key_hex, "f" * 64)
    rec.completion = "tampered"
    with pytest.raises(ValueError):
        T.verify_candidate(rec, signer.public_key_hex, "f" * 64)
    rd.write_json_once("launch.json", {"a": 1})
    with pytest.raises(FileExistsError):
        rd.write_json_once("launch.json", {"a": 2})


def test_perf_gate_budget():
    base = [T.Metrics(step=i, step_secs=1.0, grad_norm=1.0, cuda_mem_peak_used_bytes=1 << 30) for i in range(4)]
    ok = [T.Metrics(step=i, step_secs=1.05, grad_norm=1.0, cuda_mem_peak_used_bytes=(1 << 30) + (32 << 20)) for i in range(4)]
    slow = [T.Metrics(step=i, step_secs=1.2, grad_norm=1.0, cuda_mem_peak_used_bytes=1 << 30) for i in range(4)]
    fat = [T.Metrics(step=i, step_secs=1.0, grad_norm=1.0, cuda_mem_peak_used_bytes=(1 << 30) + (100 << 20)) for i in range(4)]
    assert T.compare_metrics(base, ok).passed
    assert not T.compare_metrics(base, slow).passed and not T.compare_metrics(base, fat).passed
    assert not T.compare_metrics(base, []).passed
    dead = [T.Metrics(step=i, step_secs=1.0, grad_norm=0.0, cuda_mem_peak_used_bytes=1 << 30) for i in range(4)]
    assert not T.compare_metrics(base, dead).passed
    with pytest.raises(ValueError):
        T.compare_distributed_metrics([base], [ok, ok])


# --------------------------------------------------------------- rewards
def test_countdown_math_and_data(tmp_path):
    from ferrl_b200.rewards import (CountdownProblem, CountdownReward, MathProblem, MathReward, Sample, build_prompt,
                                    generate_dataset, parse_jsonl, read_jsonl, train_eval_split, train_eval_split_by_key, DataError)
    from ferrl_b200.rewards.countdown import eval_expression
    assert generate_dataset(7, 20) == generate_dataset(7, 20) != generate_dataset(8, 20)
    assert all(1 <= p.target <= 1000 for p in generate_dataset(3, 50))
    r, p = CountdownReward(), CountdownProblem((2, 3, 4), 14)
    assert [round(r.score(p, c), 3) for c in ("<answer>2*(3+4)</answer>", "<answer>2*3+4</answer>", "<answer>2*(3+5)</answer>",
                                              "<answer>2**3</answer>", "<answer>8/(3-3)</answer>", "nothing")] == [1.0, 0.2, 0.1, 0.1, 0.1, 0.0]
    assert eval_expression("7/2*2")[0] == 7 and eval_expression("1 +") is None and eval_expression("4294967296") is None
    assert "Numbers: 2, 3, 4" in build_prompt(p) and "Target: 14" in build_prompt(p)
    m = MathReward()
    assert m.score("1,000", "so <answer> 1000 </answer>") == 1.0 and m.score("5", "<answer>6</answer>") == 0.0
    cd = read_jsonl(os.path.join(FIX, "countdown_dataset.jsonl"), CountdownProblem.from_json)
    assert len(cd) == 3 and cd[0].target.target == 100
    assert len(read_jsonl(os.path.join(FIX, "math_dataset.jsonl"), MathProblem.from_json)) >= 3
    with pytest.raises(DataError):
        parse_jsonl('{"prompt": "x"}')
    s = [Sample(f"p{i % 5}", i % 5) for i in range(12)]
    tr, ev = train_eval_split(s, 2, 1)
    assert len(tr) == 3 and len(ev) == 2 and train_eval_split(s, 2, 1)[1] == ev
    tr, ev = train_eval_split_by_key([Sample(f"p{i}", i % 3) for i in range(9)], 3, 2, lambda x: x.target)
    assert {x.target for x in tr}.isdisjoint({x.target for x in ev}) and len(ev) >= 3


def test_hf_eos_resolution_and_tokenizer(tmp_path):
    from ferrl_b200.hf import HfError, chatml, checkpoint_eos, model_vocab_size, resolve_eos
    from ferrl_b200.tokenizer import ByteTokenizer, HfTokenizer

    class Tok:
        def contains_id(self, i):
            return i < 200000
    # the committed fixtures declare no vocabulary size, which resolution needs (hf.rs: vocab_size_from_json)
    assert model_vocab_size({"vocab_size": 8, "text_config": {"vocab_size": 16}}) == 16
    for bad in ({}, {"vocab_size": 0}, {"vocab_size": "16"}):
        with pytest.raises(HfError):
            model_vocab_size(bad)
    with pytest.raises(HfError, match="vocab_size"):
        resolve_eos(os.path.join(FIX, "eos_config"), "checkpoint", None, Tok())

    def with_vocab(name):
        d = tmp_path / name
        d.mkdir()
        cfg = json.load(open(os.path.join(FIX, name, "config.json")))
        cfg["vocab_size"] = 200000
        (d / "config.json").write_text(json.dumps(cfg))
        return str(d)
    single, multi = with_vocab("eos_config"), with_vocab("eos_config_multi")
    assert checkpoint_eos(os.path.join(FIX, "eos_config")) == 151645
    assert checkpoint_eos(os.path.join(FIX, "eos_config_multi")) == [3, 4]
    with pytest.raises(HfError):
        checkpoint_eos(os.path.join(FIX, "eos_config_malformed"))
    assert resolve_eos(single, "checkpoint", None, Tok()) == 151645
    assert resolve_eos(single, "disabled", None, Tok()) is None
    with pytest.raises(HfError):
        resolve_eos(multi, "checkpoint", None, Tok())
    assert resolve_eos(multi, "explicit", 4, Tok()) == 4
    with pytest.raises(HfError):
        resolve_eos(multi, "explicit", 9, Tok())
    assert chatml("sys", "hi") == "<|im_start|>system\nsys<|im_end|>\n<|im_start|>user\nhi<|im_end|>\n<|im_start|>assistant\n"
    bt = ByteTokenizer()
    assert bt.decode(bt.encode("héllo")) == "héllo"
    ht = HfTokenizer.from_file(os.path.join(FIX, "tiny_tokenizer.json"))
    ids = ht.encode("hello world")
    assert isinstance(ids, list) and ht.vocab_size() > 0 and isinstance(ht.decode(ids), str)


# --------------------------------------------------------------- sandbox
def test_local_sandbox_limits_and_sealed_assets(tmp_path):
    from ferrl_b200.sandbox import (ApptainerSandbox, LocalSandbox, ResourceLimits, RunSpec, Verdict, make_scratch, sealed_memfd)
    sb = LocalSandbox()
    out = sb.run(RunSpec("", ["sh", "-c", "echo hi; exit 3"]))
    assert (out.verdict, out.exit_code, out.stdout) == (Verdict.EXITED, 3, b"hi\n")
    t0 = time.time()
    assert sb.run(RunSpec("", ["sh", "-c", "sleep 30 & sleep 30"], limits=ResourceLimits(wall_secs=0.4))).verdict is Verdict.TIMEOUT
    assert time.time() - t0 < 10
    d = make_scratch(str(tmp_path))
    o = sb.run(RunSpec("", ["sh", "-c", f"dd if=/dev/zero of={d}/x bs=1M count=40 2>/dev/null; sleep 5"], scratch_dir=d,
                       scratch_max_bytes=8 << 20, limits=ResourceLimits(wall_secs=10)))
    assert o.verdict is Verdict.SCRATCH_EXCEEDED
    big = sb.run(RunSpec("", ["sh", "-c", "head -c 3000000 /dev/zero"]))
    assert big.truncated and len(big.stdout) == 1 << 20
    fd = sealed_memfd("asset", b"payload")
    with pytest.raises(OSError):
        os.write(fd, b"x")
    assert os.pread(fd, 7, 0) == b"payload"
    os.close(fd)
    argv = ApptainerSandbox().build_argv(RunSpec("img.sif", ["python", "x.py"], gpu=True))
    for flag in ("--userns", "--containall", "--no-home", "--cleanenv", "--no-privs", "--nv", "--net"):
        assert flag in argv
    assert argv[argv.index("--network") + 1] == "none" and "--nv" not in ApptainerSandbox().build_argv(RunSpec("i", ["x"]))


def test_trimul_reward_shaping_and_executor_socket(tmp_path):
    from ferrl_b200.rewards.trimul import (SubmissionExtractMode, TrimulCase, TrimulReward, TrimulRewardProfile,
                                           extract_submission, parse_eval_log, render_spec)
    from ferrl_b200.sandbox import FakeSandbox, LocalSandbox, RunSpec, SandboxOutcome, Verdict
    from ferrl_b200.verifier_executor import VerifierExecutorSandbox, serve_verifier_executor
    assert extract_submission("x\n```python\nprint(1)\n```\n") == "print(1)"
    assert extract_submission("```py\na\n``` trailing") is None and extract_submission("no fence") is None
    assert extract_submission("```\na\n```</think>```\nb\n```", SubmissionExtractMode.THINKING_AFTER_THINK) == "b"
    assert render_spec([TrimulCase(32, 1, 16, 8, 5)]) == "seqlen: 32; bs: 1; dim: 16; hiddendim: 8; seed: 5; nomask: 1; distribution: normal"
    good = "test-count: 2\ntest.0.status: pass\ntest.1.status: pass\ncheck: pass\ntest-exit: 0\nbenchmark-count: 1\nbenchmark.0.mean: 2000000\nbenchmark-exit: 0\n"
    half = "test-count: 2\ntest.0.status: pass\ntest.1.status: fail\ncheck: fail\ntest-exit: 1\n"
    forged = good.replace("2000000", "5")
    logs = {"good": good, "half": half, "forged": forged}
    sb = FakeSandbox(lambda spec: SandboxOutcome(Verdict.EXITED, 0, logs[open(spec.binds[2].host).read().strip()].encode(), b""))
    r = TrimulReward(sb, "img", str(tmp_path), [TrimulCase(32, 1, 16, 8, 1)], baseline_ns=4e6)
    outs = r.reward_group_detailed(None, [f"```python\n{k}\n```" for k in ("good", "half", "forged")] + ["nothing"])
    assert abs(outs[0].reward - 3.0) < 1e-6 and outs[0].diagnostic is None          # 1.0 + min(4e6/2e6, cap 2)
    assert abs(outs[1].reward - (0.05 + 0.75 * 0.5)) < 1e-6 and outs[1].diagnostic == "trimul:test_process_failed"
    assert outs[2].reward == 0.0 and outs[3].diagnostic == "trimul:no_submission"
    assert sb.calls[0].gpu and sb.calls[0].binds[0].read_only
    with pytest.raises(ValueError):
        TrimulRewardProfile(format_extracted=0.2).validate()
    from ferrl_b200.rewards.trimul import run_status_label
    from ferrl_b200.sandbox import SandboxOutcome, Verdict
    labels = [run_status_label(SandboxOutcome(v, c, b"", b"")) for v, c in
              ((Verdict.TIMEOUT, 124), (Verdict.SIGNALED, 137), (Verdict.EXITED, 3), (Verdict.SCRATCH_EXCEEDED, 125))]
    assert labels == ["timed_out", "signaled_9", "exited_3", "scratch_exceeded"]          # trimul.rs:3293-3300
    timeout_eval = parse_eval_log("", False, labels[0])
    assert r.reward_from_extracted_eval(timeout_eval) == r.profile.format_extracted and r.diagnostic(timeout_eval) == "trimul:sandbox_timed_out"
    # a parsed grade cannot survive a sandbox failure (trimul.rs:4457-4480)
    forged = parse_eval_log("test-count: 1\ntest.0.status: pass\ncheck: pass\ntest-exit: 0\n--- benchmark ---\n"
                            "benchmark-count: 1\nbenchmark.0.mean: 500000.0\nbenchmark-exit: 0\n", False, "timed_out")
    assert r.reward_from_eval(forged) == 0.0 and r.diagnostic(forged) == "trimul:sandbox_timed_out"
    sock = str(tmp_path / "ve.sock")
    ready = threading.Event()
    t = threading.Thread(target=serve_verifier_executor, args=(sock, LocalSandbox()), kwargs=dict(max_requests=1, ready=ready))
    t.start()
    ready.wait(10)
    out = VerifierExecutorSandbox(sock).run(RunSpec("", ["sh", "-c", "echo served"]))
    t.join(10)
    assert out.ok and out.stdout == b"served\n"


# ---------------------------------------------------- artifact / orchestration
def test_artifact_audit_decision_and_manifest_last(tmp_path):
    from ferrl_b200 import artifact as A
    assert A.acceptance_from_speedups([1.05] * 9 + [1.0, 0.9]).accepted
    assert not A.acceptance_from_speedups([1.05] * 8 + [1.0] * 3).accepted
    assert not A.acceptance_from_speedups([1.02] * 11).accepted                   # strictly greater
    assert not A.acceptance_from_speedups([1.05] * 10).accepted and not A.acceptance_from_speedups([1.05] * 10 + [float("nan")]).accepted
    sched = A.audit_schedule("00" + "a" * 62)
    assert sched[0] == "reference" and sched[1] == "candidate" and len(sched) == 11 and A.audit_schedule("01" + "a" * 62)[0] == "candidate"
    run = tmp_path / "run"
    os.makedirs(run)
    json.dump({"run_id": "r1", "launch_sha256": "e" * 64}, open(run / "launch.json", "w"))
    man = A.publish_trimul_artifact(str(run), str(tmp_path / "out"), "def k(): pass", 2.5, lambda s, seed: True,
                                    lambda s, first: (1000.0, 900.0))
    assert man.accepted and man.decision["observed_material_wins"] == 11 and os.path.exists(tmp_path / "out" / A.MANIFEST_FILE)
    with pytest.raises(A.ArtifactError):
        A.publish_trimul_artifact(str(run), str(tmp_path / "out"), "x", 1.0, lambda s, seed: True, lambda s, f: (1, 1))
    rej = A.publish_trimul_artifact(str(run), str(tmp_path / "out2"), "x", 1.0, lambda s, seed: False, lambda s, f: (1000.0, 1.0))
    assert not rej.accepted and rej.blocks == []

    def crash(s, first):
        raise RuntimeError("gpu fell over")
    with pytest.raises(RuntimeError):
        A.publish_trimul_artifact(str(run), str(tmp_path / "out3"), "x", 1.0, lambda s, seed: True, crash)
    assert not os.path.exists(tmp_path / "out3" / A.MANIFEST_FILE) and os.path.exists(tmp_path / "out3" / A.ATTEMPT_FILE)


def test_orchestrated_train_report_and_perf_gate_cli(tmp_path, capsys):
    from ferrl_b200 import cli
    from ferrl_b200.orchestration import evaluate_run_health, load_and_rank_candidates, run_cli_train_setup
    from ferrl_b200.tokenizer import SyntheticTokenizer
    cfg = RunConfig.from_json({"task": "countdown", "model_dir": os.path.join(FIX, "tiny_qwen3"), "out_dir": str(tmp_path),
                               "policy": {"lora_rank": 4, "lora_alpha": 8.0}, "data": {"train_n": 8, "eval_n": 2},
                               "trainer": {"steps": 2, "group_size": 4, "max_new_tokens": 5, "checkpoint_every": 1,
                                           "candidate_log_top_k": 2, "eos_token_id": "none", "truncation_masking": False}})
    out = run_cli_train_setup(cfg, allow_dirty=True, tokenizer=SyntheticTokenizer(32, 4, 8))
    assert out.stop == "completed" and out.steps_run == 2 and out.eval_report is not None
    for f in ("launch.json", "config.json", "metrics.jsonl", "candidates.jsonl", "eval-report.json", "checkpoints"):
        assert os.path.exists(os.path.join(out.run_dir, f))
    ranked = load_and_rank_candidates(out.run_dir)
    assert len(ranked) == 4 and ranked[0].reward >= ranked[-1].reward
    from ferrl_b200.orchestration import OrchestrationError
    cpath = os.path.join(out.run_dir, "candidates.jsonl")
    good_text = open(cpath).read()
    lines = good_text.splitlines()
    bounds = dict(steps=2, group_size=4, max_new_tokens=5, rank=0, world_size=1)
    assert len(load_and_rank_candidates(out.run_dir, **bounds)) == 4
    for kw, msg in ((dict(bounds, steps=1), "coordinates exceed the launch config"),
                    (dict(bounds, max_new_tokens=1), "outside the launch-bound range"),
                    (dict(bounds, world_size=2), "rank/world disagree"),
                    (dict(bounds, require_complete=True), "expected complete logging of 8")):
        with pytest.raises(OrchestrationError, match=msg):
            load_and_rank_candidates(out.run_dir, **kw)
    for text, msg in ((good_text + lines[0] + "\n", "duplicates a training position"),
                      (good_text.rstrip("\n"), "unterminated final row"),
                      (lines[0] + "\n\n" + "\n".join(lines[1:]) + "\n", "blank row 2"),
                      (good_text + "{not json\n", "malformed")):
        open(cpath, "w").write(text)
        with pytest.raises(OrchestrationError, match=msg):
            load_and_rank_candidates(out.run_dir)
    bad = json.loads(lines[0])
    bad["reward"] = 99.0
    open(cpath, "w").write("\n".join([json.dumps(bad)] + lines[1:]) + "\n")
    with pytest.raises(OrchestrationError, match="failed launch authentication"):
        load_and_rank_candidates(out.run_dir)
    assert cli.main(["report", out.run_dir, "--json"]) in (0, 1)
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["steps"] == 2
    assert cli.main(["perf-gate", "--baseline", out.run_dir, "--candidate", out.run_dir, "--no-memory"]) in (0, 1)
    rep = evaluate_run_health([T.Metrics(step=i, reward_mean=0.0, dropped_rows=3) for i in range(4)],
                              {"reward_collapse": {"window": 3, "min": 0.1, "action": "fail"}, "dropped_rows": {"max": 5, "action": "warn"}})
    assert rep.verdict == "fail" and {f.rule for f in rep.findings} == {"reward_collapse", "dropped_rows"}


def test_preflight_with_fake_cuda():
    from ferrl_b200.preflight import PreflightError, check_device

    class Props:
        name, total_memory, multi_processor_count = "Fake", 1 << 30, 148

    class Fake:
        def __init__(self, cap, n=2, peer=True):
            self.cap, self.n, self.peer = cap, n, peer
        is_available = lambda self: self.n > 0                    # noqa: E731
        device_count = lambda self: self.n                        # noqa: E731
        get_device_capability = lambda self, i: self.cap          # noqa: E731
        get_device_properties = lambda self, i: Props             # noqa: E731
        can_device_access_peer = lambda self, a, b: self.peer     # noqa: E731
    assert check_device(0, probe=Fake((10, 0))).sm_count == 148
    for probe, kind, kw in ((Fake((9, 0)), "wrong_arch", {}), (Fake((10, 0), n=0), "no_device", {}),
                            (Fake((10, 0), peer=False), "no_peer_access", {"need_peers": 2})):
        with pytest.raises(PreflightError) as e:
            check_device(0, probe=probe, **kw)
        assert e.value.kind == kind


def test_glu_row_order_interleaves_gate_and_up():
    """Interleaved [gate | up] layout read by the GEMM's GLU epilogue: 8 gate rows, then the 8 up rows
    of the same features; applying it to a weight and splitting 16-row groups recovers both halves."""
    import torch
    from ferrl_b200.models.lora import FusedLoraLinear
    F = 24
    perm = FusedLoraLinear.glu_row_order(F)
    assert perm.tolist()[:16] == list(range(8)) + list(range(F, F + 8))
    assert sorted(perm.tolist()) == list(range(2 * F))
    w = torch.arange(2 * F * 3, dtype=torch.float32).view(2 * F, 3)
    wi = w.index_select(0, perm).view(-1, 2, 8, 3)
    assert torch.equal(wi[:, 0].reshape(F, 3), w[:F]) and torch.equal(wi[:, 1].reshape(F, 3), w[F:])
    x = torch.randn(5, 3)
    y = x @ w.index_select(0, perm).t()
    inv = torch.argsort(perm)
    assert torch.allclose(y.index_select(-1, inv), x @ w.t())


def test_gloo_rank_leaves_between_steps_is_detected(tmp_path):
    """Failure detection without a GPU: rank 1 completes a step and exits; rank 0's next collective ends
    with a typed communication error after the short process-group timeout, and the communicator stays
    poisoned so that no later step can run on half a job."""
    import subprocess
    import sys
    code = (
        "import sys, torch\n"
        "from ferrl_b200.comm import TorchDistComm, CommError, CommPoisoned\n"
        "c = TorchDistComm.bootstrap(backend='gloo', timeout_s=4)\n"
        "t = [torch.ones(2)]; c.all_reduce_sum(t); assert t[0].tolist() == [2.0, 2.0]\n"
        "c.barrier()\n"
        "if c.rank == 1:\n"
        "    print('LEFT', flush=True); sys.exit(0)\n"
        "try:\n"
        "    c.all_reduce_sum([torch.ones(2)])\n"
        "    print('NO_ERROR', flush=True); sys.exit(3)\n"
        "except CommError as e:\n"
        "    print('DETECTED', type(e).__name__, flush=True)\n"
        "try:\n"
        "    c.barrier()\n"
        "    print('NOT_POISONED', flush=True); sys.exit(4)\n"
        "except CommPoisoned:\n"
        "    print('POISONED', flush=True)\n"
        "import os; os._exit(0)\n")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = []
    for r in range(2):
        env = dict(os.environ, RANK=str(r), WORLD_SIZE="2", LOCAL_RANK=str(r), MASTER_ADDR="127.0.0.1", MASTER_PORT="29643",
                   PYTHONPATH=root)
        procs.append(subprocess.Popen([sys.executable, "-c", code], env=env, stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True))
    outs = [p.communicate(timeout=180) for p in procs]
    assert "LEFT" in outs[1][0]
    assert procs[0].returncode == 0, outs[0][1][-2000:]
    assert "DETECTED" in outs[0][0] and "POISONED" in outs[0][0], outs[0][0] + outs[0][1][-1500:]


def test_run_health_policy_rules_coverage_and_validation():
    from ferrl_b200 import run_health as H
    from ferrl_b200 import telemetry as T
    from ferrl_b200.config import ConfigError, TrainerConfig

    def rows(n, **kw):
        return [T.Metrics(step=i, reward_mean=0.5, grad_norm=1.0, rollout_capture_tokens=8, **kw) for i in range(n)]

    def cand(step, prompt, g, md):
        return T.CandidateRecord(step, 0, 1, prompt, g, 0.0, 3, "x", reward_metadata=md)

    # trailing-window MEAN, and a window that has not filled yet is reported rather than passed
    r = rows(4)
    r[-1].reward_mean = 0.0
    rule = {"reward_collapse": {"window": 2, "min": 0.3, "action": "warn"}}
    rep = H.evaluate_run_health(r, rule)
    assert rep.verdict == "warn" and "0.250000" in rep.findings[0].message
    assert H.evaluate_run_health(rows(4), rule).verdict == "ok"
    assert "only 1 metric rows" in H.evaluate_run_health(rows(1), rule).findings[0].message
    # gradient spike against the median of the positive norms; zero-gradient steps do not drag the median
    g = rows(6)
    g[0].grad_norm, g[3].grad_norm = 0.0, 9.0
    rep = H.evaluate_run_health(g, {"grad_spike": {"factor": 5.0, "action": "fail"}})
    assert rep.is_fail() and "at step 3 was 9.00x" in rep.findings[0].message and rep.render().startswith("run health policy - FAIL")
    assert H.evaluate_run_health(g, {"grad_spike": {"factor": 9.0, "action": "fail"}}).verdict == "ok"
    # dark telemetry: every step captured nothing
    dark = [T.Metrics(step=i, reward_mean=0.5) for i in range(3)]
    assert H.evaluate_run_health(dark, {"telemetry_dark": "warn"}).findings[0].rule == "telemetry_dark"
    assert H.evaluate_run_health(rows(3), {"telemetry_dark": "warn"}).verdict == "ok"
    # a non-finite metric always fails
    bad = rows(2)
    bad[1].loss = float("nan")
    assert H.evaluate_run_health(bad, {}).findings[0].rule == "non_finite"

    # candidate-based rules: full coverage of (prompt groups per step) x (group size) is required
    cc = {"correctness_collapse": {"window": 2, "min": 0.5, "action": "fail"}}
    full = [cand(s, p, g, {"correct": (s == 0), "source_sha256": "aa" if g else "bb"})
            for s in range(2) for p in (10 + s, 20 + s) for g in range(2)]
    kw = dict(group_size=2, prompt_groups_per_step=2)
    assert H.evaluate_run_health(rows(2), cc, full, **kw).verdict == "ok"                      # 4/8 = 0.5, not below
    worse = [cand(c.step, c.prompt_index, c.group_index, {"correct": False}) if i == 0 else c for i, c in enumerate(full)]
    assert "3/8 = 0.375" in H.evaluate_run_health(rows(2), cc, worse, **kw).findings[0].message
    assert "unavailable" in H.evaluate_run_health(rows(2), cc, None, **kw).findings[0].message
    assert "is empty" in H.evaluate_run_health(rows(2), cc, [], **kw).findings[0].message
    assert "missing rows for trailing metric steps 1" in \
        H.evaluate_run_health(rows(2), cc, [c for c in full if c.step == 0], **kw).findings[0].message
    assert "lacks full group coverage for trailing metric steps 1" in \
        H.evaluate_run_health(rows(2), cc, full[:-1], **kw).findings[0].message
    nometa = [cand(c.step, c.prompt_index, c.group_index, None) for c in full]
    assert "no candidate correctness metadata" in H.evaluate_run_health(rows(2), cc, nometa, **kw).findings[0].message
    tri = T.CandidateRecord(0, 0, 1, 1, 0, 0.0, 3, "x", reward_metadata={"task": "trimul", "submission_extracted": False})
    assert H.candidate_correctness(tri) is False and H.candidate_source_bucket(tri) == H.UNKNOWN_SOURCE
    sd = {"source_dominance": {"max_fraction": 0.5, "action": "warn"}}
    assert H.evaluate_run_health(rows(2), sd, full, **kw).verdict == "ok"                      # aa and bb split 4/4
    mono = [cand(c.step, c.prompt_index, c.group_index, {"source_sha256": "aa"}) for c in full]
    assert "dominant candidate source aa covered 8/8" in H.evaluate_run_health(rows(2), sd, mono, **kw).findings[0].message

    # validation
    t = TrainerConfig(steps=4, group_size=4, candidate_log_top_k=4)
    H.validate_run_health({"reward_collapse": {"window": 4, "min": 0.0, "action": "fail"}, "telemetry_dark": "warn", **cc, **sd}, t)
    for bad_rules, msg in (
            ({"reward_collapse": {"window": 5, "min": 0.0, "action": "fail"}}, "must be <= trainer.steps"),
            ({"reward_collapse": {"window": 0, "min": 0.0, "action": "fail"}}, "window must be >= 1"),
            ({"reward_collapse": {"window": 1, "min": 0.0, "action": "stop"}}, "reserved"),
            ({"reward_collapse": {"window": 1, "min": 0.0}}, "exactly the fields"),
            ({"correctness_collapse": {"window": 1, "min": 1.5, "action": "warn"}}, r"in \[0, 1\]"),
            ({"grad_spike": {"factor": 0.0, "action": "warn"}}, "factor must be finite and > 0"),
            ({"source_dominance": {"max_fraction": 2.0, "action": "warn"}}, "max_fraction"),
            ({"dropped_rows": {"max": -1, "action": "warn"}}, "non-negative"),
            ({"telemetry_dark": "stop"}, "reserved"),
            ({"surprise": 1}, "unknown field")):
        with pytest.raises(ConfigError, match=msg):
            H.validate_run_health(bad_rules, t)
    with pytest.raises(ConfigError, match="candidate_log_top_k >= trainer.group_size"):
        H.validate_run_health(sd, TrainerConfig(steps=4, group_size=4, candidate_log_top_k=2))


def test_protected_output_socket_mapping_single_connection_cap_and_executor(tmp_path):
    from ferrl_b200.sandbox import (Bind, LocalSandbox, ProtectedOutput, RunSpec, SandboxError,
                                    validate_protected_output_mapping)
    from ferrl_b200.verifier_executor import VerifierExecutorSandbox, serve_verifier_executor
    d = str(tmp_path / "scratch")
    os.mkdir(d)
    po = ProtectedOutput(d + "/grade.sock", "/scratch/grade.sock", max_bytes=64)

    def spec(code, binds=None, po=po):
        return RunSpec("", [sys.executable, "-c", code], binds=binds if binds is not None else [Bind(d, "/scratch", False)],
                       protected_output=po)
    assert validate_protected_output_mapping(spec("")) == (0, "grade.sock")
    for bad_spec, msg in (
            (spec("", binds=[Bind(d, "/scratch", True)]), "does not map through a read-write bind"),
            (spec("", binds=[Bind(d, "/scratch", False), Bind(d, "/scratch", False)]), "more than one"),
            (spec("", po=ProtectedOutput(d + "/../x.sock", "/scratch/x.sock")), "without '.' or '..'"),
            (spec("", po=ProtectedOutput(d, "/scratch")), "must name a file beneath"),
            (spec("", po=ProtectedOutput(d + "/a.sock", "/scratch/b.sock")), "does not map through")):
        with pytest.raises(SandboxError, match=msg):
            LocalSandbox().run(bad_spec)
    send = ("import os,socket,time\ns=socket.socket(socket.AF_UNIX)\ns.connect(os.environ['FERRL_GRADE_SOCKET'])\n"
            "s.sendall(b'grade: 1\\n')\n")
    # the first connection is the only one: the name is gone once it is accepted
    out = LocalSandbox().run(spec(send + "time.sleep(0.5)\nprint(os.path.exists(os.environ['FERRL_GRADE_SOCKET']))\ns.close()\n"))
    assert out.ok and out.protected_output == b"grade: 1\n" and out.stdout.strip() == b"False"
    assert os.listdir(d) == []
    # nothing connected: an empty grade, not a fallback to standard output
    out = LocalSandbox().run(spec("print('grade: 1')"))
    assert out.ok and out.protected_output == b"" and out.stdout == b"grade: 1\n"
    # the byte cap
    out = LocalSandbox().run(spec(send + "s.sendall(b'x' * 1000)\ns.close()\n"))
    assert len(out.protected_output) == 64 and out.truncated
    # through the executor service the grade travels back with the outcome
    sock = str(tmp_path / "ve.sock")
    ready = threading.Event()
    t = threading.Thread(target=serve_verifier_executor, args=(sock, LocalSandbox()), kwargs=dict(max_requests=1, ready=ready))
    t.start()
    ready.wait(10)
    out = VerifierExecutorSandbox(sock).run(spec(send + "s.close()\n"))
    t.join(10)
    assert out.ok and out.protected_output == b"grade: 1\n"


def test_preflight_driver_compat_and_error_translation():
    from ferrl_b200.preflight import PreflightError, check_driver_compat, translate_cuda_error
    assert check_driver_compat(12090) == (12, 9) and check_driver_compat(13000) == (13, 0)
    for v, kind in ((12040, "driver_too_old"), (11080, "driver_too_old"), (0, "no_driver"), (None, "no_driver")):
        with pytest.raises(PreflightError) as e:
            check_driver_compat(v)
        assert e.value.kind == kind
    cases = {"CUDA error: no kernel image is available for execution on the device": "wrong_arch",
             "the provided PTX was compiled with an unsupported toolchain.": "driver_too_old",
             "CUDA driver version is insufficient for CUDA runtime version": "driver_too_old",
             "peer access is not supported between these two devices": "no_peer_access",
             "CUDA out of memory. Tried to allocate 2.00 GiB": "out_of_memory"}
    for msg, kind in cases.items():
        assert translate_cuda_error(msg).kind == kind
    assert translate_cuda_error("an illegal memory access was encountered") is None


def test_cli_report_policy_strict_and_world_max_perf_gate(tmp_path, capsys):
    import ferrl_b200.cli as cli
    from ferrl_b200 import telemetry as T

    def write(path, rows):
        os.makedirs(os.path.dirname(path), exist_ok=True)
        w = T.MetricsWriter(path)
        for m in rows:
            w.append(m)

    def rows(secs, peak=1 << 30, n=3):
        return [T.Metrics(step=i, reward_mean=0.4, grad_norm=1.0, step_secs=secs, tokens_per_sec=10.0,
                          cuda_mem_peak_used_bytes=peak, rollout_capture_tokens=4) for i in range(n)]
    b0, b1 = str(tmp_path / "b/r0/metrics.jsonl"), str(tmp_path / "b/r1/metrics.jsonl")
    c0, c1 = str(tmp_path / "c/r0/metrics.jsonl"), str(tmp_path / "c/r1/metrics.jsonl")
    write(b0, rows(1.0)), write(b1, rows(1.0)), write(c0, rows(1.0)), write(c1, rows(1.3))
    # rank 0 alone looks fine; the job as a whole is 30 % slower because rank 1 is
    assert cli.main(["perf-gate", "--baseline", b0, "--candidate", c0, "--json"]) == 0
    capsys.readouterr()
    args = ["perf-gate", "--baseline", b0, "--baseline", b1, "--candidate", c0, "--candidate", c1]
    assert cli.main(args) == 2                                          # several paths need the world-max mode
    assert cli.main(args + ["--distributed-world-max", "--distributed-world-size", "3"]) == 2
    capsys.readouterr()
    assert cli.main(args + ["--distributed-world-max", "--distributed-world-size", "2", "--json"]) == 1
    rep = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert rep["candidate_mean_step_secs"] == pytest.approx(1.3) and "exceeds budget" in rep["failures"][0]
    assert cli.main(args + ["--distributed-world-max", "--distributed-world-size", "2",
                            "--max-step-secs-regression-pct", "40"]) == 0
    # memory: the largest rank peak counts, within slack
    write(str(tmp_path / "m/r1/metrics.jsonl"), rows(1.0, peak=(1 << 30) + (200 << 20)))
    assert cli.main(["perf-gate", "--baseline", b0, "--baseline", b1, "--candidate", c0, "--candidate",
                     str(tmp_path / "m/r1/metrics.jsonl"), "--distributed-world-max", "--distributed-world-size", "2"]) == 1
    # a rank that logged fewer steps is a failure of its own
    write(str(tmp_path / "s/r1/metrics.jsonl"), rows(1.0, n=2))
    r = T.compare_world_max_metrics([T.read_metrics(b0), T.read_metrics(b1)],
                                    [T.read_metrics(c0), T.read_metrics(str(tmp_path / "s/r1/metrics.jsonl"))])
    assert not r.passed and any("logged 2 steps" in f for f in r.failures)
    capsys.readouterr()
    # report: a metrics file is accepted; the configured policy is applied; --strict exits 2 on findings
    cfgp = tmp_path / "run.json"
    cfgp.write_text(json.dumps({"task": "countdown", "model_dir": "x", "trainer": {"steps": 3, "group_size": 4},
                                "run_health": {"reward_collapse": {"window": 2, "min": 0.9, "action": "warn"}}}))
    assert cli.main(["report", b0, "--json"]) == 0
    assert json.loads(capsys.readouterr().out.strip().splitlines()[-1])["steps"] == 3
    assert cli.main(["report", b0, "--config", str(cfgp), "--json"]) == 0           # a warning is not a failure
    js = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert js["run_health"]["verdict"] == "warn" and js["run_health"]["findings"][0]["rule"] == "reward_collapse"
    assert cli.main(["report", b0, "--config", str(cfgp), "--strict"]) == 2
    assert "run health policy - WARN" in capsys.readouterr().out


def test_verifier_executor_serves_only_the_configured_client_uid(tmp_path):
    from ferrl_b200.sandbox import LocalSandbox, RunSpec, Verdict
    from ferrl_b200.verifier_executor import VerifierExecutorSandbox, serve_verifier_executor
    sock = str(tmp_path / "ve.sock")

    def serve(uid, n):
        ready = threading.Event()
        t = threading.Thread(target=serve_verifier_executor, args=(sock, LocalSandbox()),
                             kwargs=dict(max_requests=n, ready=ready, client_uid=uid, socket_mode=0o600))
        t.daemon = True
        t.start()
        ready.wait(10)
        return t
    t = serve(os.getuid(), 1)
    assert (os.stat(sock).st_mode & 0o777) == 0o600
    out = VerifierExecutorSandbox(sock).run(RunSpec("", ["sh", "-c", "echo mine"]))
    t.join(10)
    assert out.ok and out.stdout == b"mine\n"
    # a service configured for another UID hangs up on us without running anything
    t = serve(os.getuid() + 12345, 1)
    # ... which the client reports as an infrastructure failure (nothing was learned about the command)
    from ferrl_b200.sandbox import SandboxInfrastructureError
    with pytest.raises(SandboxInfrastructureError) as e:
        VerifierExecutorSandbox(sock, timeout=5).run(RunSpec("", ["sh", "-c", "echo intruder"]))
    assert e.value.verdict is Verdict.LAUNCH_FAILED


def test_cli_trimul_score_prompt_copy_secret_seed_normalization_and_records(tmp_path, capsys, monkeypatch):
    import hashlib
    import ferrl_b200.cli as cli
    from ferrl_b200.rewards.trimul import TrimulCase, TrimulReward
    from ferrl_b200.sandbox import FakeSandbox, SandboxOutcome, Verdict
    good = "test-count: 1\ntest.0.status: pass\ncheck: pass\ntest-exit: 0\nbenchmark-count: 1\nbenchmark.0.mean: 2000000\nbenchmark-exit: 0\n"
    specs = []

    def fake(spec):
        specs.append(open(spec.binds[3].host).read())                 # the sealed test spec
        return SandboxOutcome(Verdict.EXITED, 0, good.encode(), b"")
    reward = TrimulReward(FakeSandbox(fake), "img", str(tmp_path), [TrimulCase(32, 1, 16, 8, 11), TrimulCase(64, 1, 16, 8, 11)],
                          baseline_ns=4e6)
    monkeypatch.setattr(cli, "_trimul_reward", lambda cfg: reward)
    prompt = tmp_path / "prompt.txt"
    prompt.write_text("write a kernel")
    (tmp_path / "prompt.sha256").write_text(hashlib.sha256(b"write a kernel").hexdigest() + "\n")
    cfgp = tmp_path / "run.json"
    cfgp.write_text(json.dumps({"task": "trimul", "model_dir": "x", "trainer": {"steps": 1, "group_size": 2},
                                "trimul": {"secret_seed": 11, "prompt_path": str(prompt), "image": "img"}}))
    comp = tmp_path / "c.txt"
    comp.write_text("```python\nprint(1)\n```\n [end of text]\n")
    jl = tmp_path / "c.jsonl"
    jl.write_text(json.dumps({"completion": "no code here", "step": 3, "group_index": 5, "metadata": {"k": 1}}) + "\n")
    base = ["score", "--config", str(cfgp), "--prompt-copy", str(prompt), "--completion", str(comp),
            "--completions-jsonl", str(jl), "--completion-normalization", "llama-cpp", "--model-family", "qwen3"]
    out = str(tmp_path / "scores.jsonl")
    assert cli.main(base + ["--out", out, "--score-secret-seed", "11"]) == 2          # the training seed is refused
    assert "differ from trimul.secret_seed" in capsys.readouterr().err
    assert cli.main(base + ["--out", out, "--score-secret-seed", str(1 << 32)]) == 2
    (tmp_path / "prompt.sha256").write_text("0" * 64 + "\n")
    assert cli.main(base + ["--out", out, "--score-secret-seed", "77"]) == 2
    assert "prompt copy hash mismatch" in capsys.readouterr().err and not specs
    (tmp_path / "prompt.sha256").write_text(hashlib.sha256(b"write a kernel").hexdigest() + "\n")
    assert cli.main(base + ["--out", out, "--score-secret-seed", "77"]) == 0
    summary = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert summary["scored"] == 2 and summary["positive"] == 1 and summary["diagnostics"] == {"trimul:no_submission": 1}
    assert "seed: 77;" in specs[0] and "seed: 78;" in specs[0] and "seed: 11;" not in specs[0]
    recs = [json.loads(line) for line in open(out)]
    assert recs[0]["completion"] == "```python\nprint(1)\n```\n" and abs(recs[0]["reward"] - 3.0) < 1e-6
    assert recs[0]["input_metadata"]["completion_normalization"] == {
        "mode": "llama-cpp", "changed": True, "raw_len_bytes": len(comp.read_text().encode()),
        "raw_sha256": hashlib.sha256(comp.read_text().encode()).hexdigest()}
    assert recs[0]["external_score"]["score_secret_seed"] == 77 and recs[0]["external_score"]["model_family"] == "qwen3"
    assert recs[1]["step"] == 3 and recs[1]["group_index"] == 5 and recs[1]["reward"] == 0.0
    assert recs[1]["input_metadata"]["k"] == 1 and recs[1]["input_metadata"]["completion_normalization"]["changed"] is False
    assert cli.main(base + ["--out", out, "--score-secret-seed", "77"]) == 2          # never overwritten
    assert cli.normalize_completion("abc [end of text]", "none") == ("abc [end of text]", False)


def test_cli_audit_pairs_reference_and_candidate_per_block_and_honours_inspection(tmp_path, capsys, monkeypatch):
    import ferrl_b200.cli as cli
    from ferrl_b200 import telemetry as T
    from ferrl_b200.artifact import audit_schedule
    from ferrl_b200.rewards.trimul import TrimulCase, TrimulReward
    from ferrl_b200.sandbox import FakeSandbox, SandboxOutcome, Verdict
    run = tmp_path / "run"
    run.mkdir()
    signer = T.CandidateSigner("ab" * 32)
    (run / "launch.json").write_text(json.dumps({"run_id": "r1", "launch_sha256": "ab" * 32,
                                                 "candidate_public_key": signer.public_key_hex,
                                                 "launch_authentication": "signed"}))
    (run / "config.json").write_text(json.dumps({"task": "trimul", "model_dir": "x", "trainer": {"steps": 2, "group_size": 2},
                                                 "trimul": {"secret_seed": 5, "prompt_path": "p", "image": "img"}}))
    w = T.CandidateWriter(str(run / "candidates.jsonl"), signer)
    w.append(T.CandidateRecord(0, 0, 1, 0, 0, 2.5, 9, "```python\n# FAST\n```"))
    w.append(T.CandidateRecord(1, 0, 1, 1, 1, 1.0, 9, "```python\n# SLOW\n```"))
    slow_sha = [c for c in T.read_candidates(str(run / "candidates.jsonl")) if "SLOW" in c.completion][0].record_sha256
    order = []

    def fake(spec):
        code = open(spec.binds[2].host).read()
        who = "fast" if "FAST" in code else "slow" if "SLOW" in code else "reference"
        order.append(who)
        ns = {"fast": 1000000, "slow": 2100000, "reference": 2000000}[who]
        log = f"test-count: 1\ntest.0.status: pass\ncheck: pass\ntest-exit: 0\nbenchmark-count: 1\nbenchmark.0.mean: {ns}\nbenchmark-exit: 0\n"
        return SandboxOutcome(Verdict.EXITED, 0, log.encode(), b"")
    monkeypatch.setattr(cli, "_trimul_reward", lambda cfg: TrimulReward(FakeSandbox(fake), "img", str(tmp_path),
                                                                         [TrimulCase(32, 1, 16, 8, 5)]))
    out = tmp_path / "audit-fast"
    assert cli.main(["audit", "--run-dir", str(run), "--out", str(out), "--source-inspection", "clean",
                     "--audit-cuda-visible-device", "0"]) == 0
    res = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert res["accepted"] and res["wins"] == 11
    man = json.load(open(out / "artifact-manifest.json"))
    sched = audit_schedule(man["audit_id"])
    pairs = [tuple(order[1 + 2 * i: 3 + 2 * i]) for i in range(11)]                # order[0] is the correctness re-check
    assert order[0] == "fast" and all(p == (("reference", "fast") if f == "reference" else ("fast", "reference"))
                                      for p, f in zip(pairs, sched))
    assert all(abs(b["paired_speedup"] - 2.0) < 1e-9 for b in man["blocks"])
    assert "accepted: at least nine of eleven" in open(out / "artifact-report.md").read()
    assert cli.main(["audit", "--run-dir", str(run), "--out", str(out)]) == 2      # the output is never reused
    # a named row: the slower candidate loses every pair
    assert cli.main(["audit", "--run-dir", str(run), "--candidate-sha256", slow_sha, "--out", str(tmp_path / "audit-slow")]) == 1
    assert json.load(open(tmp_path / "audit-slow" / "artifact-manifest.json"))["decision"]["observed_material_wins"] == 0
    assert cli.main(["audit", "--run-dir", str(run), "--candidate-sha256", "00" * 32, "--out", str(tmp_path / "x")]) == 1
    # a suspicious source inspection vetoes a candidate that wins every pair
    assert cli.main(["audit", "--run-dir", str(run), "--out", str(tmp_path / "audit-sus"), "--source-inspection", "suspicious",
                     "--source-inspection-notes", "reads /proc/self/environ"]) == 1
    assert "rejected: source inspection found" in open(tmp_path / "audit-sus" / "artifact-report.md").read()


def test_cli_trimul_baseline_times_the_packaged_reference_submission(tmp_path, capsys, monkeypatch):
    import ferrl_b200.cli as cli
    from ferrl_b200.rewards.trimul import TrimulCase, TrimulReward, default_eval_dir
    from ferrl_b200.sandbox import FakeSandbox, SandboxOutcome, Verdict
    seen = []

    def fake(spec):
        seen.append(open(spec.binds[2].host).read())
        log = "test-count: 1\ntest.0.status: pass\ncheck: pass\ntest-exit: 0\nbenchmark-count: 2\nbenchmark.0.mean: 1000000\nbenchmark.1.mean: 4000000\nbenchmark-exit: 0\n"
        return SandboxOutcome(Verdict.EXITED, 0, log.encode(), b"")
    monkeypatch.setattr(cli, "_trimul_reward", lambda cfg: TrimulReward(FakeSandbox(fake), "img", default_eval_dir(),
                                                                         [TrimulCase(32, 1, 16, 8, 5)]))
    cfgp = tmp_path / "run.json"
    cfgp.write_text(json.dumps({"task": "trimul", "model_dir": "x", "trainer": {"steps": 1, "group_size": 2},
                                "trimul": {"prompt_path": "p", "image": "img"}}))
    assert cli.main(["trimul-baseline", "--config", str(cfgp)]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["correct"] and out["baseline_ns"] == pytest.approx(2000000.0)       # geometric mean of the cases
    assert seen[0] == open(os.path.join(default_eval_dir(), "reference_submission.py")).read()
    with pytest.raises(SystemExit):
        cli.main(["verifier-executor", "--socket", str(tmp_path / "s.sock")])      # --client-uid is mandatory


class _FakeHeap:
    """Stands in for the symmetric heap on CPU ranks: buffers are plain host tensors, the one-shot
    all-reduce goes through the rank's communicator, and the status word can be made to report a
    peer wait that ran out."""

    def __init__(self, comm, device, wait_limit_s):
        from ferrl_b200.parallel.symm import SymmBuffer
        self._SymmBuffer = SymmBuffer
        self.comm, self.device = comm, torch.device("cpu")
        self.rank, self.world = comm.rank, comm.world_size
        self.wait_limit_s, self.poisoned = wait_limit_s, None
        self.reduces = self.checks = 0
        self.fail_check = False

    def alloc(self, nbytes):
        return self._SymmBuffer(torch.zeros((nbytes + 255) // 256 * 256, dtype=torch.uint8), [0] * self.world)

    def guard(self):
        pass

    def all_reduce_(self, buf, out):
        self.reduces += 1
        staged = buf.local.view(out.dtype)[:out.numel()].view(out.shape).to(torch.float32).clone()
        self.comm.all_reduce_sum([staged])
        out.copy_(staged.to(out.dtype))
        return out

    def check(self, what):
        self.checks += 1
        if self.fail_check:
            from ferrl_b200.comm import CommTimeout
            self.poisoned = what
            raise CommTimeout(f"{what}: kernel reported status 4 (peer wait timed out)")

    def close(self):
        pass


def _tp_cfg(tmp_path, rank, **trainer):
    t = {"steps": 2, "group_size": 4, "max_new_tokens": 4, "eos_token_id": "none", "truncation_masking": False,
         "prompts_per_item": 1}
    t.update(trainer)
    return RunConfig.from_json({"task": "countdown", "model_dir": os.path.join(FIX, "tiny_qwen3"), "out_dir": str(tmp_path),
                                "launch_authentication": "unsigned_development",
                                "policy": {"lora_rank": 4, "lora_alpha": 8.0}, "data": {"train_n": 8, "eval_n": 0},
                                "tensor_parallel": {"enabled": True, "rank": rank, "world_size": 2}, "trainer": t})


def test_train_verb_with_tensor_parallel_reaches_the_registered_peer_memory_reducer(tmp_path):
    """``tensor_parallel.enabled`` makes the train verb build the peer-memory runtime and register its
    reducers for the tensor-parallel communicator: every row-parallel reduction of rollout, scoring and
    backward goes through them (here a fake heap on two thread ranks), the status word is checked once
    per step, and the result equals the run over the plain ``Comm`` seam."""
    from ferrl_b200.comm import run_ranks
    from ferrl_b200.orchestration import run_cli_train_setup
    from ferrl_b200.parallel import symm
    from ferrl_b200.tokenizer import SyntheticTokenizer
    heaps = {}

    def factory(comm, device, limit):
        heaps[comm.rank] = _FakeHeap(comm, device, limit)
        return heaps[comm.rank]

    def body(comm, use_fake):
        out = run_cli_train_setup(_tp_cfg(tmp_path / ("fake" if use_fake else "seam"), comm.rank), comm, allow_dirty=True,
                                  tokenizer=SyntheticTokenizer(32, 4, 8), heap_factory=factory if use_fake else None)
        assert symm.gemm_all_reducer(comm) is None and symm._REDUCERS.get(id(comm)) is None    # closed with the run
        rows = [json.loads(l) for l in open(os.path.join(out.run_dir, "metrics.jsonl"))] if comm.rank == 0 else []
        return out.steps_run, [(r["loss"], r["grad_norm"]) for r in rows]
    fake = run_ranks(2, lambda c: body(c, True), timeout=120)
    assert fake[0][0] == 2
    for r in (0, 1):
        assert heaps[r].reduces > 0 and heaps[r].checks == 2          # one status check per optimizer step
    assert heaps[0].reduces == heaps[1].reduces
    seam = run_ranks(2, lambda c: body(c, False), timeout=120)
    assert seam[0][1] == fake[0][1]                                   # same sums, same order: identical metrics


def test_train_verb_turns_a_peer_wait_timeout_into_comm_timeout_on_every_rank(tmp_path):
    from ferrl_b200.comm import CommError, run_ranks
    from ferrl_b200.orchestration import run_cli_train_setup
    from ferrl_b200.tokenizer import SyntheticTokenizer

    def factory(comm, device, limit):
        h = _FakeHeap(comm, device, limit)
        h.fail_check = comm.rank == 1          # only rank 1's kernel gave up on its peer
        return h

    def body(comm):
        with pytest.raises(CommError):
            run_cli_train_setup(_tp_cfg(tmp_path, comm.rank), comm, allow_dirty=True,
                                tokenizer=SyntheticTokenizer(32, 4, 8), heap_factory=factory)
        return True
    assert run_ranks(2, body, timeout=120) == [True, True]


def test_parallel_runtime_ignores_the_in_switch_request_off_gpu_and_composes_reducers():
    """``nvls=True`` only takes effect for CUDA ranks; on CPU ranks the runtime keeps the plain reducers.  The
    composed reducer hands an input to its second member when the first declines it."""
    from ferrl_b200.comm import run_ranks
    from ferrl_b200.parallel.runtime import ParallelRuntime, _FirstOf

    def body(comm):
        rt = ParallelRuntime.create(comm, "cpu", tensor_parallel=True, hidden=64, max_rows=8,
                                    heap_factory=lambda c, d, l: _FakeHeap(c, d, l), nvls=True)
        kind = type(rt.all_reducer).__name__
        notes = list(rt.notes)
        rt.close()
        return kind, notes
    for kind, notes in run_ranks(2, body, timeout=60):
        assert kind == "SymmAllReducer" and any("peer-memory" in n for n in notes)
    calls = []
    first = lambda x: (calls.append("first"), None if x.numel() % 2 else x + 1)[1]    # noqa: E731
    second = lambda x: (calls.append("second"), x + 2)[1]                              # noqa: E731
    both = _FirstOf(first, second)
    assert torch.equal(both(torch.zeros(4)), torch.ones(4)) and calls == ["first"]
    assert torch.equal(both(torch.zeros(3)), torch.full((3,), 2.0)) and calls == ["first", "first", "second"]


def test_preflight_stage_checks_samples_and_tokenization():
    """Engine preflight (reference: crates/ferrl/src/orchestration.rs:2027-2082 and its unit tests at :6139-6168):
    exact sample bytes, a prompt that encodes to nothing is refused on every rank, ranks must hold the same samples."""
    from ferrl_b200.comm import CommMismatch, PeerFailure, SoloComm, run_ranks
    from ferrl_b200.orchestration import (OrchestrationError, exact_execution_samples, preflight_prompt_tokenization,
                                          preflight_samples)
    from ferrl_b200.rewards import Sample

    class OneToken:
        def encode(self, text):
            return [1]

    class Empty:
        def encode(self, text):
            return []

    samples = [Sample("alpha", (1, 2)), Sample("beta", {"k": [3, 4]})]
    blob = exact_execution_samples(samples)
    assert json.loads(blob.decode()) == [{"prompt": "alpha", "target": [1, 2]}, {"prompt": "beta", "target": {"k": [3, 4]}}]
    with pytest.raises(OrchestrationError, match="strict JSON cannot carry"):
        exact_execution_samples([Sample("x", float("nan"))])
    preflight_prompt_tokenization([Sample("", None), Sample("", None)], "ordered held-out samples", OneToken())
    with pytest.raises(OrchestrationError, match="ordered training samples prompt at index 0 encoded to zero tokens"):
        preflight_prompt_tokenization([Sample("", None)], "ordered training samples", Empty())
    a, b = preflight_samples(samples, samples[:1], OneToken(), SoloComm())
    assert len(a) == 64 and len(b) == 64 and a != b

    def rank_fn(comm):
        # rank 1's tokenizer yields nothing: both ranks must stop with the coordinated failure
        try:
            preflight_samples(samples, [], Empty() if comm.rank == 1 else OneToken(), comm)
        except PeerFailure as e:
            first = "local" if e.local is not None else "peer"
        else:
            first = "none"
        # rank 1 holds different samples: consensus on the digest fails on both
        try:
            preflight_samples(samples if comm.rank == 0 else samples[::-1], [], OneToken(), comm)
        except CommMismatch:
            return first, "mismatch"
        return first, "agreed"
    assert run_ranks(2, rank_fn) == [("peer", "mismatch"), ("local", "mismatch")]


def test_sequence_parallel_key_reaches_the_model_or_is_refused(tmp_path):
    """``tensor_parallel.sequence_parallel`` is part of the strict schema; a policy without a sequence-sharded form
    refuses it on every rank; the Gemma and dense families train with it over two thread ranks and end with the
    same metrics as the replicated layout (same sums in the same rank order)."""
    from ferrl_b200.comm import run_ranks
    from ferrl_b200.orchestration import OrchestrationError, run_cli_train_setup
    from ferrl_b200.tokenizer import SyntheticTokenizer

    from test_models_oracle import make_ckpt
    gemma_dir = tmp_path / "gemma_ckpt"
    gemma_dir.mkdir()
    make_ckpt(str(gemma_dir))                    # 4 query / 2 kv heads: shards over two ranks

    def cfg(root, rank, model, on):
        c = _tp_cfg(root, rank)
        c.model_dir = str(gemma_dir) if model == "gemma" else os.path.join(FIX, model)
        c.tensor_parallel.sequence_parallel = on
        return c
    assert RunConfig.from_json(cfg(tmp_path, 0, "gemma", True).to_json()).tensor_parallel.sequence_parallel is True
    with pytest.raises(Exception, match="sequence_paralel"):
        RunConfig.from_json({"task": "countdown", "model_dir": "x", "trainer": {"steps": 1},
                             "tensor_parallel": {"sequence_paralel": True}})

    def refused(comm):
        # a policy object without the sequence-sharded form (here: the attribute removed from a loaded model)
        from ferrl_b200.models.loader import LoaderOpts, load_auto_policy
        model, ident = load_auto_policy(os.path.join(FIX, "tiny_qwen3"), LoaderOpts(tp=(comm.rank, comm.world_size)))
        del model.sequence_parallel
        with pytest.raises(OrchestrationError, match="sequence_parallel is not supported"):
            run_cli_train_setup(cfg(tmp_path / "other", comm.rank, "tiny_qwen3", True), comm, allow_dirty=True,
                                tokenizer=SyntheticTokenizer(32, 4, 8), model_and_identity=(model, ident))
        return True
    assert run_ranks(2, refused, timeout=120) == [True, True]

    def train(comm, on, model):
        out = run_cli_train_setup(cfg(tmp_path / (model + ("_sp" if on else "_tp")), comm.rank, model, on), comm, allow_dirty=True,
                                  tokenizer=SyntheticTokenizer(16, 4, 8))      # the smaller vocabulary has 16 entries
        rows = [json.loads(l) for l in open(os.path.join(out.run_dir, "metrics.jsonl"))] if comm.rank == 0 else []
        return out.steps_run, [(round(r["loss"], 5), round(r["grad_norm"], 4)) for r in rows]
    for model in ("gemma", "tiny_qwen3"):
        sharded = run_ranks(2, lambda c: train(c, True, model), timeout=180)
        plain = run_ranks(2, lambda c: train(c, False, model), timeout=180)
        assert sharded[0][0] == 2 and sharded[0][1] == plain[0][1]


def test_countdown_and_math_tasks_follow_the_reference_unit_vectors():
    """The reference's own unit cases, read as golden vectors (crates/ferrl/src/countdown.rs:662-955,
    crates/ferrl/src/math.rs:149-231): expression grammar, first-answer extraction, legality, reward tiers and
    weights, split keys that close permutation / formatting leakage between train and held-out samples."""
    from ferrl_b200.rewards import CountdownProblem, CountdownReward, MathProblem, MathReward, Sample, build_prompt
    from ferrl_b200.rewards.countdown import eval_expression, extract_answer, is_legal
    from ferrl_b200.rewards.math import math_prompt, math_split_key

    def value(text):
        return eval_expression(text)[0]
    assert value("2 + 3 * 4") == 14 and value("(2 + 3) * 4") == 20 and value("2 * (3 + 4)") == 14 and value("10 - 2 - 3") == 5
    assert value("6 / 4 * 2") == 3 and value("1 / 3") != 0 and value("8 / 2 / 2") == 2 and eval_expression("5 / 0") is None
    assert list(eval_expression("2 * (3 + 4)")[1]) == [2, 3, 4]
    for bad in ("", "   ", "2 +", "2 3", "(2 + 3", "2 + 3)", "2 ^ 3", "2 + a", "99999999999"):
        assert eval_expression(bad) is None, bad
    assert extract_answer("noise <answer> 1 + 2 </answer>").strip() == "1 + 2"
    assert extract_answer("<answer>first</answer> then <answer>second</answer>") == "first"
    assert extract_answer("no tags here") is None and extract_answer("<answer>unclosed forever") is None
    assert is_legal([2, 3, 4], [4, 2, 3]) and is_legal([5, 5, 2], [5, 2, 5])
    assert not is_legal([2, 3], [2, 3, 4]) and not is_legal([2, 3, 3], [2, 3, 4])
    p = CountdownProblem((2, 3, 4), 14)
    assert p.check("2 * (3 + 4)")
    for wrong in ("2 + 3 + 4", "2 * 7", "2 * (3 + 4", "2 * 3 * 4 * 1"):
        assert not p.check(wrong), wrong
    assert "Numbers: 6, 3, 7" in build_prompt(CountdownProblem((6, 3, 7), 16)) and "Target: 16" in build_prompt(CountdownProblem((6, 3, 7), 16))
    r, s = CountdownReward(), Sample(build_prompt(p), p)
    parroted = "<answer>2 * (3 + 4)</answer>\n\nNumbers: 1, 1, 1\nTarget: 3\n<answer>1 + 1 + 1</answer>"
    assert abs(r.reward(s, parroted) - 1.0) < 1e-6
    assert r.reward(s, "I think it is 2 * 7") == 0.0
    assert r.reward(s, "<answer>2 * </answer>") == 0.1 and r.reward(s, "<answer>2 * 7</answer>") == 0.1
    assert abs(r.reward(s, "<answer>2 + 3 + 4</answer>") - 0.2) < 1e-6
    assert abs(r.reward(s, "reason... <answer>2 * (3 + 4)</answer>") - 1.0) < 1e-6
    s5 = Sample("x", CountdownProblem((5, 5, 2), 12))
    got = r.reward_group(s5, ["<answer>5 + 5 + 2</answer>", "<answer>5 + 5</answer>", "no answer"])
    assert abs(got[0] - 1.0) < 1e-6 and abs(got[1] - 0.1) < 1e-6 and got[2] == 0.0
    w = CountdownReward(format_reward=0.05, legal_reward=0.25, correct_reward=0.7)
    assert abs(w.reward(s, "<answer>2 + 3 + 4</answer>") - 0.30) < 1e-6 and abs(w.reward(s, "<answer>2 * (3 + 4)</answer>") - 1.0) < 1e-6
    assert CountdownProblem((2, 3, 4), 14).split_key() == CountdownProblem((4, 2, 3), 14).split_key()
    m = MathReward()
    q = Sample("2 + 3 = ?", MathProblem("5"))
    assert m.reward(q, "the sum is <answer>5</answer>") == 1.0 and m.reward(q, "<answer>6</answer>") == 0.0
    assert m.score("5", "the answer is <answer>5") == 0.0 and m.score("5", "the answer is 5") == 0.0
    assert m.score("1234", "<answer>1, 234</answer>") == 1.0 and m.score("1234", "<answer> 1234 </answer>") == 1.0
    assert m.score("5", "<answer>4</answer> ... <answer>5</answer>") == 0.0
    assert MathReward(correct_reward=2.5).score("42", "<answer>42</answer>") == 2.5
    assert "What is 6 * 7?" in math_prompt("What is 6 * 7?") and "<answer></answer>" in math_prompt("What is 6 * 7?")
    assert json.loads(Sample("q", MathProblem("99")).key()) == {"prompt": "q", "target": {"answer": "99"}}
    assert math_split_key(Sample("What is 1, 000 + 234?", MathProblem("1,234"))) == \
        math_split_key(Sample("What is 1000 + 234?", MathProblem(" 1234 ")))
    assert m.score("12", "<answer>1\x0b2</answer>") == 0.0          # a vertical tab is not ASCII whitespace there


def test_checkpoint_eos_resolution_follows_the_reference_unit_vectors(tmp_path):
    """crates/ferrl/src/hf.rs:516-660 read as golden cases: strict default needs exactly one declared id, an explicit
    id may fill in or override a scalar but must be a member of a declared list, the id must lie inside the model
    vocabulary and be known to the tokenizer, and ``None`` is not the same resolution as id 0."""
    from ferrl_b200.comm import run_ranks
    from ferrl_b200.hf import HfError, resolve_eos, validate_resolved_eos_consensus

    class Tok:
        def __init__(self, ids):
            self.ids = set(ids)

        def contains_id(self, i):
            return i in self.ids

    def ckpt(name, cfg):
        d = tmp_path / name
        d.mkdir()
        (d / "config.json").write_text(json.dumps(cfg))
        return str(d)
    tok = Tok(range(4))
    missing = ckpt("missing", {"vocab_size": 4})
    with pytest.raises(HfError, match="declares no eos_token_id"):
        resolve_eos(missing, "checkpoint", None, tok)
    assert resolve_eos(missing, "disabled", None, tok) is None
    assert resolve_eos(missing, "explicit", 3, tok) == 3
    multi = ckpt("multi", {"vocab_size": 4, "eos_token_id": [2, 3]})
    with pytest.raises(HfError, match="multiple EOS ids"):
        resolve_eos(multi, "checkpoint", None, tok)
    assert resolve_eos(multi, "explicit", 3, tok) == 3
    with pytest.raises(HfError, match="not a member"):
        resolve_eos(multi, "explicit", 1, tok)
    assert resolve_eos(ckpt("scalar", {"vocab_size": 4, "eos_token_id": 2}), "explicit", 3, tok) == 3
    with pytest.raises(HfError, match="EOS id 4 is not present in the loaded tokenizer vocabulary"):
        resolve_eos(ckpt("membership", {"vocab_size": 5, "eos_token_id": 4}), "checkpoint", None, tok)
    with pytest.raises(HfError, match="outside model vocab_size 4"):
        resolve_eos(ckpt("bound", {"vocab_size": 4, "eos_token_id": 4}), "checkpoint", None, Tok(range(5)))
    nested = ckpt("nested", {"eos_token_id": 1, "text_config": {"eos_token_id": 2, "vocab_size": 4}})
    assert resolve_eos(nested, "checkpoint", None, tok) == 2              # the nested text config wins

    def body(comm):
        try:
            validate_resolved_eos_consensus(0 if comm.rank == 0 else None, comm)
        except HfError:
            return "refused"
        return "accepted"
    assert run_ranks(2, body) == ["refused", "refused"]


def test_run_config_launch_rules_follow_the_reference(tmp_path):
    """crates/ferrl/src/bin/ferrl.rs:1260-1380: LoRA scale in the base dtype, tasks that need training samples, the
    TriMul seeds and isolation-tier keys, and the held-out reward on its own hidden inputs."""
    from ferrl_b200.config import ConfigError

    def cfg(**over):
        base = {"task": "countdown", "model_dir": "/m", "trainer": {"steps": 2}}
        base.update(over)
        return RunConfig.from_json(base)
    with pytest.raises(ConfigError, match="invalid policy LoRA scale: lora scale .* compute dtype BF16"):
        cfg(policy={"lora_rank": 1, "lora_alpha": 1e-42, "base_dtype": "bf16"})
    cfg(policy={"lora_rank": 1, "lora_alpha": 1e-42, "base_dtype": "f32"})
    with pytest.raises(ConfigError, match="requires data.train_n >= 1"):
        cfg(data={"train_n": 0})
    with pytest.raises(ConfigError, match="group_size = 1 requires a live data-parallel world"):
        cfg(trainer={"steps": 2, "group_size": 1, "reward_group_scope": "distributed_same_prompt"})
    tri = {"prompt_path": "p", "image": "i"}
    for extra, msg in (({"secret_seed": 2 ** 32}, "secret_seed must be between 0 and 4294967295"),
                       ({"held_out_secret_seed": 5}, "held_out_secret_seed requires data.eval_n >= 1"),
                       ({"verifier_executor_socket": "/s"}, "valid only with \"dedicated_uid_service_v1\""),
                       ({"verifier_apptainer_bin": "apptainer"}, "must be an absolute path"),
                       ({"verifier_isolation_tier": "dedicated_uid_service_v1", "verifier_apptainer_bin": "/usr/bin/apptainer"},
                        "valid only with \"same_uid_apptainer_v1\"")):
        with pytest.raises(ConfigError, match=msg):
            cfg(task="trimul", trimul=dict(tri, **extra), data={"train_n": 4, "eval_n": 0})
    with pytest.raises(ConfigError, match="held-out eval requires trimul.held_out_secret_seed"):
        cfg(task="trimul", trimul=tri, data={"train_n": 4, "eval_n": 2})
    with pytest.raises(ConfigError, match="differ from trimul.secret_seed"):
        cfg(task="trimul", trimul=dict(tri, secret_seed=7, held_out_secret_seed=7), data={"train_n": 4, "eval_n": 2})
    prompt = tmp_path / "prompt.txt"
    prompt.write_text("write a kernel")
    from ferrl_b200.orchestration import build_task
    good = cfg(task="trimul", data={"train_n": 4, "eval_n": 2},
               trimul={"prompt_path": str(prompt), "image": "img.sif", "secret_seed": 7, "held_out_secret_seed": 1000})
    train, held, reward = build_task(good)
    assert len(train) == 4 and len(held) == 2
    assert [c.seed for c in reward.cases] == [7] and [c.seed for c in reward.held_out_reward.cases] == [1000]
    assert reward.held_out_reward is not reward and reward.held_out_reward.image == reward.image


def test_in_image_script_and_verifier_entry_protocol(tmp_path):
    """crates/ferrl/src/sandbox.rs:1560-1650, 1738-1790, 1910-1936 as golden cases: the Apptainer argument vector,
    the in-image script (mandatory ulimits, entry marker, quoted words) and the rule that a run which ends before
    the marker is an infrastructure failure, not a verdict about the command."""
    import dataclasses

    from ferrl_b200 import sandbox as S
    spec = S.RunSpec("/img.sif", ["python", "/work/eval.py"], binds=[S.Bind("/h/ref", "/ref", True), S.Bind("/h/scratch", "/work", False)],
                     workdir="/work", env=[("PYTHONHASHSEED", "0")])
    argv = S.ApptainerSandbox("apptainer").build_argv(spec)
    for flag in ("--userns", "--containall", "--no-home", "--cleanenv", "--no-eval", "--disable-cache", "--no-mount",
                 "--no-privs", "--drop-caps"):
        assert flag in argv
    assert argv[argv.index("--no-mount") + 1] == "home,cwd,hostfs,bind-paths" and argv[argv.index("--drop-caps") + 1] == "all"
    assert any(argv[i:i + 3] == ["--net", "--network", "none"] for i in range(len(argv)))
    assert "--nv" not in argv and "--nv" in S.ApptainerSandbox("apptainer").build_argv(dataclasses.replace(spec, gpu=True))
    host_net = S.ApptainerSandbox("apptainer").build_argv(dataclasses.replace(spec, network=S.NetworkPolicy.HOST))
    assert "--net" not in host_net and "--network" not in host_net
    assert "/h/ref:/ref:ro" in argv and "/h/scratch:/work:rw" in argv
    assert argv[argv.index("--pwd") + 1] == "/work" and argv[argv.index("--env") + 1] == "PYTHONHASHSEED=0"
    assert argv[-4:-1] == ["/img.sif", "/bin/bash", "-c"] and "exec 'python'" in argv[-1]

    limited = dataclasses.replace(spec, limits=S.ResourceLimits(wall_secs=30, cpu_secs=25, address_space=2 << 30, max_procs=64,
                                                               max_file=8 << 20))
    script = S._in_container_script(limited)
    for piece in ("ulimit -t 25", "ulimit -v 2097152", "ulimit -u 64", "ulimit -f 8192", S.SANDBOX_ENTRY_MARKER,
                  "exec 'python' '/work/eval.py'"):
        assert piece in script
    assert script.count("|| exit 114") == 4 and script.startswith("umask 077; ") and "timeout" not in script
    bare = dataclasses.replace(spec, limits=S.ResourceLimits(wall_secs=5, cpu_secs=None, address_space=None, max_procs=None,
                                                            max_file=None))
    assert S._in_container_script(bare) == \
        f"umask 077; printf '%s\\n' '{S.SANDBOX_ENTRY_MARKER}' >&2; exec 'python' '/work/eval.py'"
    assert S.shell_quote("a b") == "'a b'" and S.shell_quote("it's") == "'it'\\''s'"
    assert "'python' '/work/a b.py'" in S._in_container_script(S.RunSpec("/img.sif", ["python", "/work/a b.py"]))

    # entered, then the command itself fails: an ordinary outcome with the marker removed from stderr
    sb = S.LocalSandbox()
    out = sb.run(S.RunSpec("none", ["/bin/sh", "-c", "printf oops >&2; exit 7"], limits=S.ResourceLimits(wall_secs=10)))
    assert out.verdict is S.Verdict.EXITED and out.exit_code == 7 and out.stderr == b"oops"

    class BrokenWrapper(S.LocalSandbox):
        def _payload_argv(self, spec):
            return ["/bin/sh", "-c", "printf wrapper-failed >&2; exit 7"]
    with pytest.raises(S.SandboxInfrastructureError) as e:
        BrokenWrapper().run(S.RunSpec("none", ["true"], limits=S.ResourceLimits(wall_secs=10)))
    assert e.value.exit_code == 7 and e.value.stderr == b"wrapper-failed" and "before verifier entry" in str(e.value)
    # callers that run something other than a verifier may waive the protocol
    out = BrokenWrapper().run(S.RunSpec("none", ["true"], limits=S.ResourceLimits(wall_secs=10), require_entry_marker=False))
    assert out.exit_code == 7 and out.stderr == b"wrapper-failed"

    # a verifier that never started must not score the candidate: the reward raises instead of returning 0
    from ferrl_b200.rewards import RewardError
    from ferrl_b200.rewards.trimul import TrimulCase, TrimulReward

    class NeverEnters(S.Sandbox):
        def run(self, spec):
            raise S.SandboxInfrastructureError(S.Verdict.EXITED, 255, b"FATAL: container creation failed")
    reward = TrimulReward(NeverEnters(), "img.sif", str(tmp_path), [TrimulCase(32, 1, 16, 16, 1)])
    with pytest.raises(RewardError, match="infrastructure failed"):
        reward.reward(None, "```python\ndef custom_kernel(data):\n    return data\n```")


def test_dedicated_verifier_service_refuses_deployments_that_isolate_nothing(tmp_path):
    """crates/ferrl/src/verifier_executor.rs:750-788 and its unit cases: distinct non-root users, absolute paths,
    no world access to the socket, a socket parent the client cannot write."""
    from ferrl_b200.sandbox import SandboxError
    from ferrl_b200.verifier_executor import validate_service_config
    parent = tmp_path / "run"
    parent.mkdir(mode=0o755)
    ok = dict(socket_path=str(parent / "ve.sock"), work_root=str(tmp_path / "work"), client_uid=1000,
              apptainer_bin="/usr/bin/apptainer", socket_mode=0o660, service_uid=os.stat(parent).st_uid or 4242)
    if os.stat(parent).st_uid == 0:            # running as root here: play a service user that owns the directory
        os.chown(parent, 4242, -1)
    validate_service_config(**ok)
    for change, msg in ((dict(client_uid=ok["service_uid"]), "distinct non-root UIDs"), (dict(client_uid=0), "distinct non-root UIDs"),
                        (dict(service_uid=0), "distinct non-root UIDs"), (dict(socket_path="run/ve.sock"), "absolute"),
                        (dict(work_root=str(tmp_path / "a" / ".." / "work")), "absolute"),
                        (dict(apptainer_bin="apptainer"), "absolute path"), (dict(socket_mode=0o666), "no world access")):
        with pytest.raises(SandboxError, match=msg):
            validate_service_config(**dict(ok, **change))
    (parent / "ve.sock").write_text("")
    with pytest.raises(SandboxError, match="already exists"):
        validate_service_config(**ok)
    (parent / "ve.sock").unlink()
    os.chmod(parent, 0o775)
    with pytest.raises(SandboxError, match="closed to group/world writes"):
        validate_service_config(**ok)


def test_a_rank_that_cannot_load_its_policy_stops_every_rank_before_the_first_collective(tmp_path):
    """Setup stages are coordinated (crates/ferrl/src/orchestration.rs:1899-2025): one rank failing to load raises a
    coordinated failure everywhere instead of leaving its peers waiting in a collective."""
    from ferrl_b200.comm import PeerFailure, run_ranks
    from ferrl_b200.orchestration import run_cli_train_setup
    from ferrl_b200.tokenizer import SyntheticTokenizer
    import ferrl_b200.orchestration as orch
    real, who = orch.load_auto_policy, threading.local()

    def flaky(model_dir, opts):
        if who.rank == 1:
            raise OSError("shard 2 of 2 is missing")
        return real(model_dir, opts)

    def body(comm):
        who.rank = comm.rank
        try:
            run_cli_train_setup(_tp_cfg(tmp_path, comm.rank), comm, allow_dirty=True, tokenizer=SyntheticTokenizer(32, 4, 8))
        except PeerFailure as e:
            return "local" if e.local is not None else "peer"
        return "completed"
    orch.load_auto_policy = flaky
    try:
        out = run_ranks(2, body, timeout=60)
    finally:
        orch.load_auto_policy = real
    assert out == ["peer", "local"]


def test_run_directory_layout_and_reuse_rules_follow_the_reference(tmp_path):
    """crates/ferrl/src/telemetry.rs:2883-3030, 3245-3264: a fresh run directory holds exactly the checkpoints
    directory (no per-run log file), a run id is never reused, also not after a crash that left only candidate rows,
    and a run is continued only from a directory that exists."""
    rd = T.RunDir.create(str(tmp_path), "run-001")
    assert os.listdir(rd.root) == ["checkpoints"] and rd.run_id == "run-001" and not os.path.exists(rd.path("run.log"))
    T.CandidateWriter(rd.candidates_path, None).append(T.CandidateRecord(0, 0, 1, 0, 0, 1.0, 2, "candidate"))
    assert not os.path.exists(rd.metrics_path)                         # the crash-before-metrics window
    with pytest.raises(FileExistsError):
        T.RunDir.create(str(tmp_path), "run-001")
    w = T.MetricsWriter(rd.metrics_path)
    w.append(T.Metrics(step=0))
    again = T.RunDir.open(str(tmp_path), "run-001")
    assert again.root == rd.root
    T.MetricsWriter(again.metrics_path).append(T.Metrics(step=1))
    assert len(open(again.metrics_path).read().splitlines()) == 2       # open() continues the stream
    with pytest.raises(FileNotFoundError):
        T.RunDir.open(str(tmp_path), "run-nope")
    bare = tmp_path / "run-002"
    bare.mkdir()
    assert os.listdir(T.RunDir.open(str(bare)).root) == ["checkpoints"]


def test_candidate_ledger_refuses_nonfinite_rewards_and_a_second_signing_process(tmp_path):
    """crates/ferrl/src/telemetry.rs:3115-3185: nothing is written for a non-finite reward, and a launch-bound writer
    never appends to rows an earlier process signed with a key that no longer exists."""
    rd = T.RunDir.create(str(tmp_path), "run")
    plain = T.CandidateWriter(rd.candidates_path, None)
    for reward in (float("nan"), float("-inf"), float("inf")):
        with pytest.raises(ValueError, match="not finite"):
            plain.append(T.CandidateRecord(0, 0, 1, 0, 0, reward, 1, "candidate"))
    assert not os.path.exists(rd.candidates_path) or open(rd.candidates_path).read() == ""
    plain.append(T.CandidateRecord(0, 0, 1, 0, 0, 1.0, 1, "existing"))
    with pytest.raises(ValueError, match="non-empty ledger .* signing capability is unavailable"):
        T.CandidateWriter(rd.candidates_path, T.CandidateSigner("ab" * 32))
    assert len(open(rd.candidates_path).read().splitlines()) == 1


def test_countdown_generator_is_solvable_by_an_independent_solver():
    """crates/ferrl/src/countdown.rs:838-942: every generated problem is reachable by combining all numbers with
    + - * / over exact rationals (checked without the generator's own fold), also with large products, and the
    degenerate one-number configuration yields the number itself."""
    from fractions import Fraction

    from ferrl_b200.rewards.countdown import CountdownConfig, generate_dataset

    def reachable(nums):
        if len(nums) == 1:
            return {nums[0]}
        out = set()
        for i in range(len(nums)):
            for j in range(len(nums)):
                if i == j:
                    continue
                a, b = nums[i], nums[j]
                rest = [nums[k] for k in range(len(nums)) if k not in (i, j)]
                for c in [a + b, a - b, a * b] + ([a / b] if b != 0 else []):
                    out |= reachable(rest + [c])
        return out

    def solvable(p):
        return Fraction(p.target) in reachable([Fraction(n) for n in p.numbers])
    data = generate_dataset(7, 40, CountdownConfig(4, 1, 12, 200))
    assert len(data) == 40
    assert all(len(p.numbers) == 4 and all(1 <= n <= 12 for n in p.numbers) and p.target > 0 and solvable(p) for p in data)
    assert all(p.target > 0 and solvable(p) for p in generate_dataset(99, 30, CountdownConfig(4, 10, 80, 100_000)))
    assert [(p.numbers, p.target) for p in generate_dataset(1, 3, CountdownConfig(1, 5, 5, 1000))] == [((5,), 5)] * 3
    assert generate_dataset(42, 8) == generate_dataset(42, 8) != generate_dataset(43, 8)
