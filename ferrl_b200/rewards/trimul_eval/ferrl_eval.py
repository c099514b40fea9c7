"""TriMul evaluation driver: runs inside the verifier sandbox, grades one submitted kernel.

Counterpart of the reference's ``crates/ferrl/src/trimul_eval_driver.py`` (process split ``:1-11``,
candidate hardening ``:483-604``, candidate session ``:955-1108``, testing / benchmarking
``:1142-1236``).  Self-contained on purpose: the directory holding this file is bound read-only
at ``/eval`` and started as ``python -I /eval/ferrl_eval.py``; it needs only ``torch``.

Two processes.  The *parent* (this file's ``main``) owns the hidden case inputs, the fp32
reference result, the comparison, the clock and standard output - the grade log.  The *payload*
(``--payload <fd>``) imports the submission and serves ``load`` / ``run`` requests over one
socket; it starts with no inherited descriptors but that socket, with standard streams on
``/dev/null``, ``no_new_privs`` set, not dumpable, core dumps off and in its own session so its
whole tree can be killed.  Only length-prefixed raw tensor bytes with a JSON header cross the
boundary - nothing is unpickled from the payload, and no device allocation is shared.  The
timing metric covers the ``run`` request, the kernel, the device-to-host copy of its result and
the receipt of those bytes; the check of that result happens after the clock stops, and every
timed run is checked, on inputs the payload has not seen before.

Inputs (environment): ``FERRL_SUBMISSION`` (path of the candidate module, which defines
``custom_kernel(data)`` with ``data = (input, mask, weights, config)``), ``FERRL_TEST_SPEC`` and
``FERRL_BENCH_SPEC`` (one case per line: ``seqlen: N; bs: B; dim: C; hiddendim: H; seed: S;
nomask: 0|1; distribution: normal|cauchy``), optional ``FERRL_EVAL_REPS`` (timed runs per
benchmark case, default 5), ``FERRL_EVAL_CALL_TIMEOUT`` (seconds per request, default 120),
``FERRL_EVAL_DEVICE`` (``cuda`` when available, else ``cpu``).

Output (standard output, ``key: value`` lines): ``test-count``, ``test.<i>.spec``,
``test.<i>.status`` (``pass`` | ``fail`` | ``timeout``), ``test.<i>.error``, ``check``
(``pass`` | ``fail``), ``test-exit``, ``benchmark-count``, ``benchmark.<i>.runs`` / ``.mean`` /
``.std`` / ``.best`` / ``.worst`` (nanoseconds), ``benchmark-exit``, ``timing-metric``.  With
``FERRL_GRADE_SOCKET`` set, the same lines also go to that Unix socket - the protected channel the
host reads the grade from - which the parent connects before the payload process exists.
"""
import json
import math
import os
import select
import signal
import socket
import struct
import subprocess
import sys
import time

TIMING_METRIC = "isolated-payload-latency-v1"
MAX_MESSAGE_BYTES = 4 << 30
MAX_ERROR_CHARS = 240
EXIT_FAIL = 112
RTOL, ATOL = 2e-2, 2e-2
_DTYPES = ("float32", "float16", "bfloat16", "float64", "int64", "int32", "bool")


# ------------------------------------------------------------------ wire format
def pack_bundle(kind, tensors=None, meta=None):
    """``kind`` + JSON header + raw tensor bytes.  ``tensors``: name -> CPU tensor."""
    import torch
    entries, blobs = [], []
    for name, t in (tensors or {}).items():
        t = t.detach().contiguous().cpu()
        dt = str(t.dtype).replace("torch.", "")
        flat = t.reshape(-1)
        flat = flat.to(torch.uint8) if t.dtype == torch.bool else flat.view(torch.uint8)
        raw = flat.numpy().tobytes() if flat.numel() else b""
        entries.append({"name": name, "dtype": dt, "shape": list(t.shape), "nbytes": len(raw)})
        blobs.append(raw)
    head = json.dumps({"kind": kind, "meta": meta or {}, "tensors": entries}).encode()
    return struct.pack("<Q", len(head)) + head + b"".join(blobs)


def unpack_bundle(data):
    """Inverse of ``pack_bundle`` with every length checked; never unpickles."""
    import torch
    if len(data) < 8:
        raise ValueError("short message")
    (n,) = struct.unpack("<Q", data[:8])
    if n > len(data) - 8 or n > (1 << 20):
        raise ValueError("bad header length")
    head = json.loads(data[8:8 + n].decode())
    off, out = 8 + n, {}
    for e in head.get("tensors", []):
        if e["dtype"] not in _DTYPES or e["nbytes"] < 0 or off + e["nbytes"] > len(data):
            raise ValueError("bad tensor entry")
        shape = [int(d) for d in e["shape"]]
        numel = 1
        for d in shape:
            if d < 0:
                raise ValueError("negative dimension")
            numel *= d
        dt = getattr(torch, e["dtype"])
        item = 1 if dt == torch.bool else torch.empty((), dtype=dt).element_size()
        if numel * item != e["nbytes"]:
            raise ValueError("tensor bytes do not match its shape")
        raw = bytearray(data[off:off + e["nbytes"]])
        if numel == 0:
            t = torch.empty(shape, dtype=dt)
        elif dt == torch.bool:
            t = torch.frombuffer(raw, dtype=torch.uint8).to(torch.bool).reshape(shape)
        else:
            t = torch.frombuffer(raw, dtype=dt).reshape(shape).clone()
        out[str(e["name"])] = t
        off += e["nbytes"]
    return head.get("kind"), head.get("meta", {}), out


def send_msg(sock, data):
    if len(data) > MAX_MESSAGE_BYTES:
        raise ValueError("message too large")
    sock.sendall(struct.pack("<Q", len(data)) + data)


def recv_msg(sock, deadline):
    """One length-prefixed message, or ``None`` when the deadline passes or the peer is gone."""
    def read(n):
        buf = bytearray()
        while len(buf) < n:
            left = deadline - time.monotonic()
            if left <= 0:
                return None
            r, _, _ = select.select([sock], [], [], min(left, 1.0))
            if not r:
                continue
            chunk = sock.recv(min(n - len(buf), 1 << 20))
            if not chunk:
                return None
            buf += chunk
        return bytes(buf)
    head = read(8)
    if head is None:
        return None
    (n,) = struct.unpack("<Q", head)
    if n > MAX_MESSAGE_BYTES:
        return None
    return read(n)


# ------------------------------------------------------------------ the task
def parse_spec(text):
    """``seqlen: 32; bs: 1; ...`` lines -> list of dicts (unknown keys are kept as strings)."""
    cases = []
    for line in text.splitlines():
        line = line.strip()
        if not line:
            continue
        case = {}
        for part in line.split(";"):
            if ":" in part:
                k, v = part.split(":", 1)
                case[k.strip()] = v.strip()
        for k in ("seqlen", "bs", "dim", "hiddendim", "seed"):
            case[k] = int(case[k])
        case["nomask"] = bool(int(case.get("nomask", 1)))
        case["distribution"] = case.get("distribution", "normal")
        cases.append(case)
    return cases


def render_case(case):
    return "; ".join(f"{k}: {int(v) if isinstance(v, bool) else v}" for k, v in case.items())


def generate_case(case, salt=0):
    """Inputs of one case on the CPU, a pure function of ``(case, salt)``: the activation
    ``[bs, n, n, dim]``, the pair mask ``[bs, n, n]`` and the layer's weights."""
    import torch
    g = torch.Generator().manual_seed((int(case["seed"]) * 1000003 + salt * 7919 + 17) & ((1 << 63) - 1))
    bs, n, dim, hid = case["bs"], case["seqlen"], case["dim"], case["hiddendim"]
    if case["distribution"] == "cauchy":
        u = torch.rand(bs, n, n, dim, generator=g)
        x = 2.0 * torch.tan(math.pi * (u - 0.5))
    else:
        x = torch.randn(bs, n, n, dim, generator=g)
    mask = torch.ones(bs, n, n) if case["nomask"] else (torch.rand(bs, n, n, generator=g) < 0.5).float()

    def w(o, i):
        return torch.randn(o, i, generator=g) / math.sqrt(i)
    weights = {
        "norm.weight": 1.0 + 0.1 * torch.randn(dim, generator=g), "norm.bias": 0.1 * torch.randn(dim, generator=g),
        "left_proj.weight": w(hid, dim), "right_proj.weight": w(hid, dim),
        "left_gate.weight": w(hid, dim), "right_gate.weight": w(hid, dim), "out_gate.weight": w(hid, dim),
        "to_out_norm.weight": 1.0 + 0.1 * torch.randn(hid, generator=g),
        "to_out_norm.bias": 0.1 * torch.randn(hid, generator=g),
        "to_out.weight": w(dim, hid),
    }
    return x, mask, weights, {"dim": dim, "hidden_dim": hid}


def reference_trimul(x, mask, weights, config):
    """The outgoing triangle multiplicative update in fp32 (LayerNorm -> gated left/right
    projections -> sum over k of left[i,k] * right[j,k] -> LayerNorm -> output gate -> projection)."""
    import torch
    import torch.nn.functional as F
    x = x.float()
    wt = {k: v.float() for k, v in weights.items()}
    xn = F.layer_norm(x, (config["dim"],), wt["norm.weight"], wt["norm.bias"])
    m = mask.float().unsqueeze(-1)
    left = (xn @ wt["left_proj.weight"].t()) * m * torch.sigmoid(xn @ wt["left_gate.weight"].t())
    right = (xn @ wt["right_proj.weight"].t()) * m * torch.sigmoid(xn @ wt["right_gate.weight"].t())
    out_gate = torch.sigmoid(xn @ wt["out_gate.weight"].t())
    out = torch.einsum("bikd,bjkd->bijd", left, right)
    out = F.layer_norm(out, (config["hidden_dim"],), wt["to_out_norm.weight"], wt["to_out_norm.bias"])
    return (out * out_gate) @ wt["to_out.weight"].t()


def check_output(got, want):
    """``None`` when the candidate's result matches the reference, else a one-line reason."""
    import torch
    if not isinstance(got, torch.Tensor):
        return "output is not a tensor"
    if tuple(got.shape) != tuple(want.shape):
        return f"shape mismatch: got {tuple(got.shape)}, expected {tuple(want.shape)}"
    got = got.float()
    if not torch.isfinite(got).all():
        return "output contains non-finite values"
    diff = (got - want).abs()
    bad = diff > (ATOL + RTOL * want.abs())
    if bad.any():
        return f"mismatch in {int(bad.sum())} of {bad.numel()} elements, max abs error {float(diff.max()):.4g}"
    return None


def one_line(msg):
    msg = " ".join(str(msg).split())
    return msg[:MAX_ERROR_CHARS]


# ------------------------------------------------------------------ payload (untrusted side)
def _harden_payload(keep_fd):
    """Before any candidate code runs: own session, no new privileges, not dumpable, no cores,
    nothing open but the channel, standard streams on /dev/null, a scrubbed environment."""
    import ctypes
    import resource
    try:
        os.setsid()
    except OSError:
        pass
    libc = ctypes.CDLL(None, use_errno=True)
    libc.prctl(38, 1, 0, 0, 0)          # PR_SET_NO_NEW_PRIVS
    libc.prctl(4, 0, 0, 0, 0)           # PR_SET_DUMPABLE = 0
    resource.setrlimit(resource.RLIMIT_CORE, (0, 0))
    null = os.open(os.devnull, os.O_RDWR)
    for fd in (0, 1, 2):
        os.dup2(null, fd)
    os.closerange(3, keep_fd)
    os.closerange(keep_fd + 1, 4096)
    for k in list(os.environ):
        if k.startswith("FERRL_") and k not in ("FERRL_SUBMISSION", "FERRL_SCRATCH", "FERRL_EVAL_DEVICE"):
            del os.environ[k]
    scratch = os.environ.get("FERRL_SCRATCH")
    if scratch and os.path.isdir(scratch):
        os.chdir(scratch)
    return _install_syscall_filter()


def _install_syscall_filter():
    """Last hardening step: the seccomp deny list of ``syscall_filter.py`` (the file next to this one; loaded
    by path because the interpreter runs isolated).  Returns the kernel's evidence, or a record that says why
    the filter is absent (``FERRL_EVAL_SECCOMP=0``, another architecture)."""
    if os.environ.get("FERRL_EVAL_SECCOMP", "1") == "0":
        return {"seccomp_policy": None, "reason": "disabled by FERRL_EVAL_SECCOMP=0"}
    import importlib.util
    import platform
    if platform.machine() != "x86_64" or not sys.platform.startswith("linux"):
        return {"seccomp_policy": None, "reason": f"no policy for {sys.platform}/{platform.machine()}"}
    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "syscall_filter.py")
    spec = importlib.util.spec_from_file_location("ferrl_syscall_filter", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod.install()


def payload_main(fd):
    try:
        hardening = _harden_payload(fd)
    except BaseException as e:  # noqa: BLE001 - a payload that could not be confined must not run candidate code
        sock = socket.socket(fileno=fd)
        send_msg(sock, pack_bundle("error", meta={"error": one_line(f"payload hardening failed: {type(e).__name__}: {e}"),
                                                  "infrastructure": True}))
        return
    sock = socket.socket(fileno=fd)
    import importlib.machinery
    import importlib.util
    import torch
    dev = torch.device(os.environ.get("FERRL_EVAL_DEVICE") or ("cuda" if torch.cuda.is_available() else "cpu"))
    try:
        loader = importlib.machinery.SourceFileLoader("submission", os.environ["FERRL_SUBMISSION"])
        spec = importlib.util.spec_from_loader("submission", loader)
        mod = importlib.util.module_from_spec(spec)
        sys.dont_write_bytecode = True
        loader.exec_module(mod)
        kernel = getattr(mod, "custom_kernel")
        send_msg(sock, pack_bundle("ready", meta={"hardening": hardening}))
    except BaseException as e:  # noqa: BLE001 - reported to the parent as a candidate failure
        send_msg(sock, pack_bundle("error", meta={"error": one_line(f"import failed: {type(e).__name__}: {e}")}))
        return
    data = None
    forever = time.monotonic() + 10 ** 9
    while True:
        msg = recv_msg(sock, forever)
        if msg is None:
            return
        kind, meta, tensors = unpack_bundle(msg)
        try:
            if kind == "load":
                weights = {k[2:]: v.to(dev) for k, v in tensors.items() if k.startswith("w.")}
                data = (tensors["input"].to(dev), tensors["mask"].to(dev), weights, dict(meta))
                if dev.type == "cuda":
                    torch.cuda.synchronize()
                send_msg(sock, pack_bundle("loaded"))
            elif kind == "run":
                out = kernel(data)
                if not isinstance(out, torch.Tensor):
                    raise TypeError("custom_kernel must return a tensor")
                send_msg(sock, pack_bundle("result", {"output": out.detach().to("cpu")}))
            elif kind == "quit":
                return
        except BaseException as e:  # noqa: BLE001
            send_msg(sock, pack_bundle("error", meta={"error": one_line(f"{type(e).__name__}: {e}")}))


# ------------------------------------------------------------------ parent (trusted side)
class CandidateFailure(Exception):
    """The candidate failed (wrong result, exception, timeout): graded, not an infrastructure error."""

    def __init__(self, msg, timeout=False):
        super().__init__(msg)
        self.timeout = timeout


class CandidateSession:
    """One payload process and the request/response exchange with it."""

    def __init__(self, call_timeout):
        self.call_timeout = call_timeout
        ours, theirs = socket.socketpair()
        self.sock = ours
        self.proc = subprocess.Popen([sys.executable, "-I", os.path.abspath(__file__), "--payload", str(theirs.fileno())],
                                     pass_fds=[theirs.fileno()], stdin=subprocess.DEVNULL, stdout=subprocess.DEVNULL,
                                     stderr=subprocess.DEVNULL, start_new_session=True)
        theirs.close()
        self.dead = None
        kind, meta, _ = self._recv(max(call_timeout, 60.0))
        if kind != "ready":
            self.close()
            if isinstance(meta, dict) and meta.get("infrastructure"):
                raise RuntimeError(meta.get("error", "payload hardening failed"))      # not the candidate's fault
            raise CandidateFailure(meta.get("error", "payload did not start") if isinstance(meta, dict) else "payload did not start")
        self.hardening = meta.get("hardening") if isinstance(meta, dict) else None
        h = self.hardening
        if isinstance(h, dict) and h.get("seccomp_policy") is not None and (h.get("seccomp_mode") != 2 or h.get("no_new_privs") != 1):
            self.close()
            raise RuntimeError(f"payload reports an inactive syscall filter: {h}")

    def _recv(self, timeout):
        msg = recv_msg(self.sock, time.monotonic() + timeout)
        if msg is None:
            gone = self.proc.poll() is not None
            self.close()
            self.dead = "payload process exited" if gone else f"no answer within {timeout:g} s"
            raise CandidateFailure(self.dead, timeout=not gone)
        try:
            return unpack_bundle(msg)
        except (ValueError, KeyError, TypeError) as e:
            self.close()
            self.dead = f"malformed answer from the payload: {e}"
            raise CandidateFailure(self.dead) from e

    def _call(self, data, expect):
        if self.dead:
            raise CandidateFailure(self.dead)
        try:
            send_msg(self.sock, data)
        except OSError as e:
            self.close()
            self.dead = f"payload channel closed: {e}"
            raise CandidateFailure(self.dead) from e
        kind, meta, tensors = self._recv(self.call_timeout)
        if kind == "error":
            raise CandidateFailure(one_line(meta.get("error", "candidate raised")))
        if kind != expect:
            raise CandidateFailure(f"unexpected answer {kind!r}")
        return tensors

    def load(self, x, mask, weights, config):
        tensors = {"input": x, "mask": mask}
        tensors.update({"w." + k: v for k, v in weights.items()})
        self._call(pack_bundle("load", tensors, config), "loaded")

    def run(self):
        """One timed request: returns ``(output, elapsed_ns)``; the clock covers request, kernel,
        device-to-host copy and receipt, and stops before the result is decoded or checked."""
        req = pack_bundle("run")
        if self.dead:
            raise CandidateFailure(self.dead)
        t0 = time.perf_counter_ns()
        try:
            send_msg(self.sock, req)
        except OSError as e:
            self.close()
            self.dead = f"payload channel closed: {e}"
            raise CandidateFailure(self.dead) from e
        msg = recv_msg(self.sock, time.monotonic() + self.call_timeout)
        t1 = time.perf_counter_ns()
        if msg is None:
            gone = self.proc.poll() is not None
            self.close()
            self.dead = "payload process exited" if gone else f"no answer within {self.call_timeout:g} s"
            raise CandidateFailure(self.dead, timeout=not gone)
        try:
            kind, meta, tensors = unpack_bundle(msg)
        except (ValueError, KeyError, TypeError) as e:
            raise CandidateFailure(f"malformed answer from the payload: {e}") from e
        if kind == "error":
            raise CandidateFailure(one_line(meta.get("error", "candidate raised")))
        if kind != "result" or "output" not in tensors:
            raise CandidateFailure(f"unexpected answer {kind!r}")
        return tensors["output"], t1 - t0

    def close(self):
        """Kill the payload's whole session (it may have started children)."""
        if self.proc.poll() is None:
            try:
                os.killpg(self.proc.pid, signal.SIGKILL)
            except (ProcessLookupError, PermissionError):
                self.proc.kill()
        try:
            self.proc.wait(timeout=10)
        except subprocess.TimeoutExpired:
            pass
        try:
            self.sock.close()
        except OSError:
            pass


def _session(log, call_timeout):
    try:
        session = CandidateSession(call_timeout)
    except CandidateFailure as e:
        return None, e
    h = session.hardening if isinstance(session.hardening, dict) else {}
    log("payload-hardening: " + one_line(json.dumps({k: h.get(k) for k in ("seccomp_policy", "seccomp_mode", "seccomp_filters",
                                                                          "no_new_privs", "reason") if k in h}, sort_keys=True)))
    return session, None


def run_tests(log, cases, call_timeout):
    log(f"test-count: {len(cases)}")
    session, err = _session(log, call_timeout)
    passed = 0
    for i, case in enumerate(cases):
        log(f"test.{i}.spec: {render_case(case)}")
        status, msg = "fail", None
        try:
            if session is None:
                raise err
            x, mask, weights, config = generate_case(case)
            want = reference_trimul(x, mask, weights, config)
            session.load(x, mask, weights, config)
            got, _ = session.run()
            msg = check_output(got, want)
            status = "pass" if msg is None else "fail"
        except CandidateFailure as e:
            status, msg = ("timeout" if e.timeout else "fail"), str(e)
        passed += status == "pass"
        log(f"test.{i}.status: {status}")
        if msg:
            log(f"test.{i}.error: {one_line(msg)}")
    if session is not None:
        session.close()
    ok = passed == len(cases) and len(cases) > 0
    log(f"check: {'pass' if ok else 'fail'}")
    log(f"test-exit: {0 if ok else EXIT_FAIL}")
    return ok


def run_benchmarks(log, cases, call_timeout, reps):
    log(f"benchmark-count: {len(cases)}")
    log(f"timing-metric: {TIMING_METRIC}")
    session, err = _session(log, call_timeout)
    ok = session is not None
    for i, case in enumerate(cases):
        log(f"benchmark.{i}.spec: {render_case(case)}")
        times = []
        try:
            if session is None:
                raise err
            for rep in range(reps + 1):                      # rep 0 warms the candidate up, untimed
                x, mask, weights, config = generate_case(case, salt=rep + 1)
                want = reference_trimul(x, mask, weights, config)
                session.load(x, mask, weights, config)
                got, ns = session.run()
                bad = check_output(got, want)                # after the clock stopped
                if bad is not None:
                    raise CandidateFailure(f"timed run {rep} was wrong: {bad}")
                if rep > 0:
                    times.append(float(ns))
        except CandidateFailure as e:
            ok = False
            log(f"benchmark.{i}.error: {one_line(e)}")
            continue
        mean = sum(times) / len(times)
        var = sum((t - mean) ** 2 for t in times) / max(len(times) - 1, 1)
        log(f"benchmark.{i}.runs: {len(times)}")
        log(f"benchmark.{i}.mean: {mean:.1f}")
        log(f"benchmark.{i}.std: {math.sqrt(var):.1f}")
        log(f"benchmark.{i}.best: {min(times):.1f}")
        log(f"benchmark.{i}.worst: {max(times):.1f}")
    if session is not None:
        session.close()
    log(f"benchmark-exit: {0 if ok else EXIT_FAIL}")
    return ok


def main(argv=None):
    argv = sys.argv[1:] if argv is None else argv
    if len(argv) == 2 and argv[0] == "--payload":
        payload_main(int(argv[1]))
        return 0
    import ctypes
    try:
        ctypes.CDLL(None).prctl(4, 0, 0, 0, 0)               # the grader itself is not dumpable either
    except OSError:
        pass
    out = os.fdopen(os.dup(1), "w", buffering=1)
    grade = None
    path = os.environ.pop("FERRL_GRADE_SOCKET", None)
    if path:
        # the protected channel: connected before any candidate code exists in this sandbox; the
        # host stops listening after this one connection, so the grade cannot come from anyone else
        grade = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        try:
            grade.connect(path)
        except OSError as e:
            out.write(f"infrastructure-error: cannot reach the grade socket: {one_line(e)}\n")
            return 2

    def log(line):
        out.write(line + "\n")
        if grade is not None:
            grade.sendall((line + "\n").encode())
    try:
        tests = parse_spec(open(os.environ["FERRL_TEST_SPEC"]).read())
        bench_path = os.environ.get("FERRL_BENCH_SPEC")
        benches = parse_spec(open(bench_path).read()) if bench_path else []
        if not os.path.isfile(os.environ["FERRL_SUBMISSION"]):
            raise FileNotFoundError(os.environ["FERRL_SUBMISSION"])
    except (KeyError, OSError, ValueError) as e:
        log(f"infrastructure-error: {one_line(e)}")
        return 2
    call_timeout = float(os.environ.get("FERRL_EVAL_CALL_TIMEOUT", "120"))
    reps = max(1, int(os.environ.get("FERRL_EVAL_REPS", "5")))
    ok = run_tests(log, tests, call_timeout)
    if ok and benches:
        ok = run_benchmarks(log, benches, call_timeout, reps) and ok
    return 0 if ok else EXIT_FAIL


if __name__ == "__main__":
    sys.exit(main())
