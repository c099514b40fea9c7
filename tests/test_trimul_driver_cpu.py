"""The packaged TriMul evaluation driver, started the way the sandbox starts it (CPU device)."""
import os
import subprocess
import sys

import pytest
import torch

from ferrl_b200.rewards.trimul import (EVAL_DRIVER_FILE, TrimulCase, TrimulReward, default_eval_dir, parse_eval_log,
                                       render_spec)
from ferrl_b200.sandbox import FakeSandbox, SandboxOutcome, Verdict, sealed_memfd

DRIVER = os.path.join(default_eval_dir(), EVAL_DRIVER_FILE)
CASES = [TrimulCase(12, 1, 16, 8, 3), TrimulCase(8, 2, 8, 8, 4, nomask=False, distribution="cauchy")]

GOOD = '''
import torch, torch.nn.functional as F
print("check: pass")
print("benchmark.0.mean: 1")
def custom_kernel(data):
    x, mask, w, cfg = data
    xn = F.layer_norm(x, (cfg["dim"],), w["norm.weight"], w["norm.bias"])
    m = mask.unsqueeze(-1)
    l = (xn @ w["left_proj.weight"].t()) * m * torch.sigmoid(xn @ w["left_gate.weight"].t())
    r = (xn @ w["right_proj.weight"].t()) * m * torch.sigmoid(xn @ w["right_gate.weight"].t())
    og = torch.sigmoid(xn @ w["out_gate.weight"].t())
    o = torch.einsum("bikd,bjkd->bijd", l, r)
    o = F.layer_norm(o, (cfg["hidden_dim"],), w["to_out_norm.weight"], w["to_out_norm.bias"])
    return (o * og) @ w["to_out.weight"].t()
'''


def grade(tmp_path, submission, cases=CASES, bench=True, **env):
    spec = tmp_path / "tests.txt"
    spec.write_text(render_spec(cases))
    fd = sealed_memfd("submission", submission.encode())          # the candidate travels as a sealed in-memory file
    try:
        e = {"PATH": os.environ.get("PATH", ""), "FERRL_SUBMISSION": f"/proc/{os.getpid()}/fd/{fd}",
             "FERRL_TEST_SPEC": str(spec), "FERRL_SCRATCH": str(tmp_path), "FERRL_EVAL_REPS": "2", "FERRL_EVAL_DEVICE": "cpu"}
        if bench:
            e["FERRL_BENCH_SPEC"] = str(spec)
        e.update(env)
        r = subprocess.run([sys.executable, "-I", DRIVER], env=e, capture_output=True, text=True, timeout=300)
    finally:
        os.close(fd)
    return r, parse_eval_log(r.stdout)


def test_correct_submission_passes_and_is_timed_and_cannot_forge_the_grade_log(tmp_path):
    r, ev = grade(tmp_path, GOOD)
    assert r.returncode == 0, r.stdout + r.stderr
    assert ev.correct and ev.tests_total == 2 and ev.tests_passed == 2 and ev.test_exit == 0 and ev.benchmark_exit == 0
    assert len(ev.benchmark_means_ns) == 2 and all(m > 1000 for m in ev.benchmark_means_ns) and not ev.implausible()
    assert r.stdout.count("check:") == 1 and "benchmark.0.mean: 1\n" not in r.stdout    # the candidate's prints went nowhere
    assert "timing-metric: isolated-payload-latency-v1" in r.stdout
    # and through the reward: correct + speed term against a baseline
    sb = FakeSandbox(lambda spec: SandboxOutcome(Verdict.EXITED, 0, r.stdout.encode(), b""))
    rew = TrimulReward(sb, "img", default_eval_dir(), CASES, baseline_ns=ev.geomean_ns)
    out = rew.reward_group_detailed(None, [f"```python\n{GOOD}\n```"])[0]
    assert abs(out.reward - 2.0) < 1e-6 and out.diagnostic is None
    assert sb.calls[0].binds[0].host == default_eval_dir() and sb.calls[0].command[-1] == "/eval/ferrl_eval.py"


def test_packaged_reference_submission_is_correct(tmp_path):
    src = open(os.path.join(default_eval_dir(), "reference_submission.py")).read()
    r, ev = grade(tmp_path, src, bench=False)
    assert r.returncode == 0 and ev.correct and not ev.has_benchmark_section


def test_wrong_results_shapes_exceptions_and_import_failures_are_graded(tmp_path):
    wrong = GOOD.replace('@ w["to_out.weight"].t()', '@ w["to_out.weight"].t() * 1.2')
    r, ev = grade(tmp_path, wrong)
    assert r.returncode == 112 and not ev.correct and ev.tests_passed == 0 and "mismatch in" in r.stdout
    assert not ev.has_benchmark_section                                # a wrong kernel is never timed
    shape = GOOD.replace('@ w["to_out.weight"].t()', '@ w["to_out.weight"].t()[:, :4]')
    r, ev = grade(tmp_path, shape)
    assert ev.shape_failure and not ev.correct
    # correct on the first case only: partial credit is visible to the reward
    half = GOOD.replace("    x, mask, w, cfg = data\n", "    x, mask, w, cfg = data\n    assert x.shape[0] == 1, 'batched input'\n")
    r, ev = grade(tmp_path, half)
    assert ev.tests_passed == 1 and ev.tests_total == 2 and "AssertionError: batched input" in r.stdout
    r, ev = grade(tmp_path, "import does_not_exist_anywhere\n")
    assert ev.tests_passed == 0 and "import failed: ModuleNotFoundError" in r.stdout
    r, ev = grade(tmp_path, "def custom_kernel(data):\n    return 'text'\n")
    assert ev.tests_passed == 0 and "must return a tensor" in r.stdout
    # a result that is right on the test inputs but replayed on the (different) timed inputs fails the benchmark
    replay = GOOD.replace("def custom_kernel(data):", "_seen = {}\ndef _real(data):") + '''
def custom_kernel(data):
    key = tuple(data[0].shape)
    if key not in _seen or len(_seen[key]) < 2:
        _seen.setdefault(key, []).append(_real(data))
    return _seen[key][-1]
'''
    r, ev = grade(tmp_path, replay, cases=CASES[:1])
    assert ev.correct and ev.benchmark_exit == 112 and "was wrong" in r.stdout and ev.geomean_ns is None


def test_hanging_candidate_times_out_and_its_process_tree_is_killed(tmp_path):
    marker = tmp_path / "child.pid"
    hang = f'''
import os, subprocess, time
def custom_kernel(data):
    p = subprocess.Popen(["sleep", "600"])
    open({str(marker)!r}, "w").write(str(p.pid))
    time.sleep(600)
'''
    r, ev = grade(tmp_path, hang, cases=CASES[:1], FERRL_EVAL_CALL_TIMEOUT="3")
    assert r.returncode == 112 and "test.0.status: timeout" in r.stdout and not ev.correct
    pid = int(marker.read_text())
    for _ in range(50):
        if not os.path.exists(f"/proc/{pid}") or "Z" in open(f"/proc/{pid}/stat").read().split(")")[-1].split()[0]:
            break
        import time
        time.sleep(0.1)
    else:
        pytest.fail("the candidate's child survived the grader")


def test_wire_format_rejects_inconsistent_lengths():
    sys.path.insert(0, default_eval_dir())
    try:
        import ferrl_eval as E
    finally:
        sys.path.pop(0)
    msg = E.pack_bundle("result", {"output": torch.arange(6, dtype=torch.float32).reshape(2, 3)})
    kind, _, t = E.unpack_bundle(msg)
    assert kind == "result" and torch.equal(t["output"], torch.arange(6.0).reshape(2, 3))
    with pytest.raises(ValueError):
        E.unpack_bundle(msg[:-4])                                      # bytes shorter than the header claims
    with pytest.raises(ValueError):
        E.unpack_bundle(msg.replace(b'"shape": [2, 3]', b'"shape": [9, 9]'))
    with pytest.raises(ValueError):
        E.unpack_bundle(msg.replace(b'"float32"', b'"objectx"'))
    x, mask, w, cfg = E.generate_case({"seqlen": 6, "bs": 1, "dim": 8, "hiddendim": 4, "seed": 1, "nomask": False, "distribution": "normal"})
    x2 = E.generate_case({"seqlen": 6, "bs": 1, "dim": 8, "hiddendim": 4, "seed": 1, "nomask": False, "distribution": "normal"})[0]
    assert torch.equal(x, x2) and not torch.equal(x, E.generate_case({"seqlen": 6, "bs": 1, "dim": 8, "hiddendim": 4, "seed": 1, "nomask": False, "distribution": "normal"}, salt=1)[0])
    out = E.reference_trimul(x, mask, w, cfg)
    assert out.shape == x.shape and E.check_output(out.clone(), out) is None and "shape" in E.check_output(out[:, :2], out)


def test_reward_end_to_end_through_the_supervised_sandbox_and_protected_socket(tmp_path):
    """Completion -> extraction -> sealed files -> supervisor -> driver -> grade over the protected
    socket -> shaped reward.  No container here: bind names are translated to host paths."""
    from ferrl_b200.sandbox import LocalSandbox
    seen = []

    class Spy(LocalSandbox):
        def run(self, spec):
            out = super().run(spec)
            seen.append((spec, out))
            return out
    rew = TrimulReward(Spy(), "", default_eval_dir(), CASES[:1], scratch_root=str(tmp_path), gpu=False,
                       driver=(sys.executable, "-I", "/eval/ferrl_eval.py"), baseline_ns=1e12, wall_secs=240)
    cheat = "print('check: pass')\ndef custom_kernel(data):\n    return data[0] * 0\n"
    outs = rew.reward_group_detailed(None, [f"```python\n{GOOD}\n```", f"```python\n{cheat}\n```"])
    assert abs(outs[0].reward - 3.0) < 1e-6 and outs[0].diagnostic is None          # correct + capped speed term
    assert outs[1].reward == pytest.approx(rew.profile.runnable) and outs[1].diagnostic is not None
    spec, out = seen[0]
    assert out.protected_output is not None and b"check: pass" in out.protected_output
    assert spec.protected_output.sandbox_socket == "/scratch/grade.sock"
    assert os.listdir(tmp_path) == []                                  # scratch (and its socket) removed
