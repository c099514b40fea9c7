"""Process sandbox for untrusted verifier payloads.

Reference ``crates/ferrl/src/sandbox.rs``: ``RunSpec`` ``:254-343`` and
``ResourceLimits`` ``:192``; ``ApptainerSandbox::build_argv`` ``:479-527``
(user namespace, ``--containall --no-home --cleanenv --no-eval --disable-cache
--no-mount home,cwd,hostfs,bind-paths --no-privs --drop-caps all``, ``--nv``
only on request, ``--net --network none``); a host-side wall-clock supervisor
that kills the whole process tree ``:1009-1205``; a scratch byte-cap monitor
``:1216-1484``; 1 MiB capture cap ``:841``; a protected output socket on which
the in-sandbox verifier returns its grade, so that nothing the candidate prints
can pass for one ``:598-1007``; sealed in-memory assets
(``crates/ferrl/src/trimul.rs:697-840``).

The OS-level part - new session, rlimits before exec, wall clock, scratch byte
polling, group kill, reaping - is the native supervisor
``csrc/native/sandbox_launcher.cpp``; this module builds its command line,
wraps Apptainer around the payload, caps captured output and maps the
supervisor's exit codes to a ``SandboxOutcome``.  ``LocalSandbox`` runs the
payload under the supervisor without a container (tests and trusted tasks);
``FakeSandbox`` is a scripted double.
"""
from __future__ import annotations

import enum
import fcntl
import os
import shutil
import socket
import subprocess
import tempfile
import threading
from dataclasses import dataclass, field
from typing import Callable, Optional, Sequence

CAPTURE_CAP = 1 << 20
LAUNCHER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "bin", "ferrl-sandbox-launch")


class SandboxError(RuntimeError):
    pass


class SandboxInfrastructureError(SandboxError):
    """The wrapper or the container runtime failed before the command inside the image was entered: an
    infrastructure failure, never a verdict about the command (crates/ferrl/src/sandbox.rs:411-420)."""

    def __init__(self, verdict, exit_code: int, stderr: bytes):
        self.verdict, self.exit_code, self.stderr = verdict, exit_code, stderr
        super().__init__(f"sandbox infrastructure failed before verifier entry ({getattr(verdict, 'value', verdict)} "
                         f"{exit_code}): {stderr.decode(errors='replace')}")


class NetworkPolicy(str, enum.Enum):
    NONE = "none"
    HOST = "host"


@dataclass
class ResourceLimits:
    wall_secs: float = 120.0
    cpu_secs: Optional[int] = 120
    address_space: Optional[int] = None     # hostile to CUDA's huge virtual reservations: off by default
    max_procs: Optional[int] = 256
    max_file: Optional[int] = 1 << 30


@dataclass
class Bind:
    host: str
    container: str
    read_only: bool = True

    def render(self) -> str:
        return f"{self.host}:{self.container}:{'ro' if self.read_only else 'rw'}"


@dataclass
class ProtectedOutput:
    """A Unix socket the host listens on and the in-sandbox verifier connects to once to hand
    back its result.  ``host_socket`` must lie beneath the host side of exactly one read-write
    bind and ``sandbox_socket`` at the same relative path beneath that bind's container side."""
    host_socket: str
    sandbox_socket: str
    max_bytes: int = CAPTURE_CAP


PROTECTED_OUTPUT_ENV = "FERRL_GRADE_SOCKET"


@dataclass
class RunSpec:
    image: str
    command: list
    binds: list = field(default_factory=list)
    workdir: str = "/"
    env: list = field(default_factory=list)          # (key, value)
    gpu: bool = False
    network: NetworkPolicy = NetworkPolicy.NONE
    limits: ResourceLimits = field(default_factory=ResourceLimits)
    scratch_dir: Optional[str] = None
    scratch_max_bytes: Optional[int] = None
    stdin_bytes: Optional[bytes] = None
    protected_output: Optional[ProtectedOutput] = None
    # the in-image shell announces that it is about to exec the command; a run that ends without the
    # announcement failed in the wrapper or the container runtime, not in the command (see _in_container_script)
    require_entry_marker: bool = True


class Verdict(str, enum.Enum):
    EXITED = "exited"
    TIMEOUT = "timeout"
    SCRATCH_EXCEEDED = "scratch_exceeded"
    SIGNALED = "signaled"
    LAUNCH_FAILED = "launch_failed"


@dataclass
class SandboxOutcome:
    verdict: Verdict
    exit_code: int
    stdout: bytes
    stderr: bytes
    truncated: bool = False
    protected_output: Optional[bytes] = None     # what arrived on the protected socket (None: nothing connected)

    @property
    def ok(self) -> bool:
        return self.verdict is Verdict.EXITED and self.exit_code == 0


def _normal_absolute(path: str) -> bool:
    return os.path.isabs(path) and all(c not in (".", "..") for c in path.split("/")) and "//" not in path.rstrip("/")


def validate_protected_output_mapping(spec: RunSpec) -> Optional[tuple]:
    """``(bind_index, relative_path)`` of the read-write bind the protected socket travels through."""
    po = spec.protected_output
    if po is None:
        return None
    for label, p in (("protected output host socket", po.host_socket),
                     ("protected output sandbox socket", po.sandbox_socket)):
        if not _normal_absolute(p):
            raise SandboxError(f"{label} must be an absolute path without '.' or '..': {p}")
    found = []
    for i, b in enumerate(spec.binds):
        if b.read_only or not (_normal_absolute(b.host) and _normal_absolute(b.container)):
            continue
        h, c = b.host.rstrip("/") + "/", b.container.rstrip("/") + "/"
        if (po.host_socket + "/").startswith(h) and (po.sandbox_socket + "/").startswith(c):
            rh, rc = po.host_socket[len(h):], po.sandbox_socket[len(c):]
            if rh == rc:
                found.append((i, rh))
    if not found:
        raise SandboxError("protected output socket does not map through a read-write bind")
    if len(found) > 1:
        raise SandboxError("protected output socket maps through more than one read-write bind")
    if not found[0][1]:
        raise SandboxError("protected output socket must name a file beneath its read-write bind")
    return found[0]


class _ProtectedListener:
    """Accepts ONE connection on the host socket, removes the socket's name at once so no second
    party can connect, and reads until end of stream or the byte cap."""

    def __init__(self, po: ProtectedOutput):
        self.po, self.data, self.truncated = po, None, False
        if os.path.lexists(po.host_socket):
            raise SandboxError(f"protected output socket path already exists: {po.host_socket}")
        self.sock = socket.socket(socket.AF_UNIX, socket.SOCK_STREAM)
        old = os.umask(0o077)
        try:
            self.sock.bind(po.host_socket)
        finally:
            os.umask(old)
        self.sock.listen(1)
        self.sock.settimeout(0.2)
        self.stop = threading.Event()
        self.thread = threading.Thread(target=self._serve, daemon=True)
        self.thread.start()

    def _unlink(self):
        try:
            os.unlink(self.po.host_socket)
        except OSError:
            pass

    def _serve(self):
        conn = None
        while not self.stop.is_set():
            try:
                conn, _ = self.sock.accept()
                break
            except socket.timeout:
                continue
            except OSError:
                return
        self._unlink()
        if conn is None:
            return
        buf = bytearray()
        conn.settimeout(0.2)
        with conn:
            while True:
                try:
                    chunk = conn.recv(1 << 16)
                except socket.timeout:
                    if self.stop.is_set():
                        break
                    continue
                except OSError:
                    break
                if not chunk:
                    break
                buf += chunk
                if len(buf) > self.po.max_bytes:
                    self.truncated = True
                    del buf[self.po.max_bytes:]
                    break
        self.data = bytes(buf)

    def finish(self) -> Optional[bytes]:
        """Call after the sandboxed process has ended."""
        self.stop.set()
        self.thread.join(5)
        self.sock.close()
        self._unlink()
        return self.data


def sealed_memfd(name: str, data: bytes) -> int:
    """An anonymous in-memory file holding ``data`` that can no longer be written, grown,
    shrunk or re-sealed: the verifier assets a payload receives cannot be swapped under it."""
    fd = os.memfd_create(name, os.MFD_CLOEXEC | os.MFD_ALLOW_SEALING)
    try:
        os.write(fd, data)
        seals = fcntl.F_SEAL_WRITE | fcntl.F_SEAL_GROW | fcntl.F_SEAL_SHRINK | fcntl.F_SEAL_SEAL
        fcntl.fcntl(fd, fcntl.F_ADD_SEALS, seals)
    except BaseException:
        os.close(fd)
        raise
    return fd


def ensure_launcher() -> str:
    if not os.path.exists(LAUNCHER):
        from . import _build
        _build.build_launcher()
    return LAUNCHER


def _supervisor_argv(spec: RunSpec) -> list:
    lim = spec.limits
    argv = [ensure_launcher(), "--wall-ms", str(int(lim.wall_secs * 1000))]
    if lim.cpu_secs:
        argv += ["--cpu-s", str(int(lim.cpu_secs))]
    if lim.max_file:
        argv += ["--fsize", str(int(lim.max_file))]
    if lim.address_space:
        argv += ["--as", str(int(lim.address_space))]
    if spec.scratch_dir and spec.scratch_max_bytes:
        argv += ["--scratch", spec.scratch_dir, "--scratch-max", str(int(spec.scratch_max_bytes))]
    return argv


# Written to standard error by the trusted in-image shell immediately before it execs the command.  Its absence
# proves that the launcher or the container runtime failed before the command began
# (crates/ferrl/src/sandbox.rs:783-816).
SANDBOX_ENTRY_MARKER = "ferrl-sandbox-verifier-entry-v1"
ULIMIT_FAILED_EXIT = 114


def shell_quote(word: str) -> str:
    """Single-quoted shell word; an embedded quote closes, escapes and reopens the quoting."""
    return "'" + word.replace("'", "'\\''") + "'"


def _in_container_script(spec: RunSpec) -> str:
    """The ``-c`` script run inside the image: restrictive umask, the requested ``ulimit``s, the entry marker, then
    ``exec`` of the command.  A requested limit is mandatory: if the shell cannot install it, it exits (114) before
    the marker and the run counts as an infrastructure failure instead of running under a weaker policy.  The wall
    clock is not enforced here: the host-side supervisor owns it."""
    lim = spec.limits
    script = "umask 077; "
    if lim.cpu_secs is not None:
        script += f"ulimit -t {max(1, int(lim.cpu_secs))} || exit {ULIMIT_FAILED_EXIT}; "
    if lim.address_space is not None:
        script += f"ulimit -v {int(lim.address_space) // 1024} || exit {ULIMIT_FAILED_EXIT}; "
    if lim.max_procs is not None:
        script += f"ulimit -u {int(lim.max_procs)} || exit {ULIMIT_FAILED_EXIT}; "
    if lim.max_file is not None:
        script += f"ulimit -f {int(lim.max_file) // 1024} || exit {ULIMIT_FAILED_EXIT}; "
    return script + f"printf '%s\\n' '{SANDBOX_ENTRY_MARKER}' >&2; exec " + " ".join(shell_quote(c) for c in spec.command)


def consume_entry_marker(stderr: bytes) -> tuple[bytes, bool]:
    """``(stderr without the marker line, whether it was there)``."""
    token = (SANDBOX_ENTRY_MARKER + "\n").encode()
    at = stderr.find(token)
    if at < 0:
        return stderr, False
    return stderr[:at] + stderr[at + len(token):], True


def _cap(data: bytes) -> tuple[bytes, bool]:
    return (data[:CAPTURE_CAP], True) if len(data) > CAPTURE_CAP else (data, False)


def _map_exit(rc: int, out: bytes, err: bytes) -> SandboxOutcome:
    o, t1 = _cap(out)
    e, t2 = _cap(err)
    if rc == 124:
        return SandboxOutcome(Verdict.TIMEOUT, rc, o, e, t1 or t2)
    if rc == 125:
        return SandboxOutcome(Verdict.SCRATCH_EXCEEDED, rc, o, e, t1 or t2)
    if rc in (126, 127):
        return SandboxOutcome(Verdict.LAUNCH_FAILED, rc, o, e, t1 or t2)
    if rc > 128:
        return SandboxOutcome(Verdict.SIGNALED, rc, o, e, t1 or t2)
    return SandboxOutcome(Verdict.EXITED, rc, o, e, t1 or t2)


class Sandbox:
    def run(self, spec: RunSpec) -> SandboxOutcome:
        raise NotImplementedError


class _SupervisedSandbox(Sandbox):
    def _payload_argv(self, spec: RunSpec) -> list:
        raise NotImplementedError

    def _env(self, spec: RunSpec) -> dict:
        return {"PATH": "/usr/local/sbin:/usr/local/bin:/usr/sbin:/usr/bin:/sbin:/bin"}

    def run(self, spec: RunSpec) -> SandboxOutcome:
        if not spec.command:
            raise SandboxError("empty command")
        validate_protected_output_mapping(spec)
        argv = _supervisor_argv(spec) + ["--"] + self._payload_argv(spec)
        listener = _ProtectedListener(spec.protected_output) if spec.protected_output is not None else None
        try:
            out = self._run(spec, argv)
        finally:
            got = listener.finish() if listener is not None else None
        if spec.require_entry_marker:
            out.stderr, entered = consume_entry_marker(out.stderr)
            if not entered:
                raise SandboxInfrastructureError(out.verdict, out.exit_code, out.stderr)
        if listener is not None:
            out.protected_output = got if got is not None else b""     # asked for and silent: an empty grade
            out.truncated = out.truncated or listener.truncated
        return out

    def _run(self, spec: RunSpec, argv: list) -> SandboxOutcome:
        try:
            # generous outer timeout: the supervisor enforces the real limit and always returns
            res = subprocess.run(argv, input=spec.stdin_bytes, capture_output=True, env=self._env(spec),
                                 timeout=spec.limits.wall_secs + 30)
        except subprocess.TimeoutExpired as e:
            return SandboxOutcome(Verdict.TIMEOUT, 124, (e.stdout or b"")[:CAPTURE_CAP], (e.stderr or b"")[:CAPTURE_CAP])
        except OSError as e:
            return SandboxOutcome(Verdict.LAUNCH_FAILED, 126, b"", str(e).encode())
        return _map_exit(res.returncode, res.stdout, res.stderr)


class ApptainerSandbox(_SupervisedSandbox):
    def __init__(self, apptainer_bin: str = "apptainer", shell: str = "/bin/bash"):
        self.bin, self.shell = apptainer_bin, shell

    def available(self) -> bool:
        return shutil.which(self.bin) is not None

    def build_argv(self, spec: RunSpec) -> list:
        a = ["exec", "--userns", "--containall", "--no-home", "--cleanenv", "--no-eval", "--disable-cache",
             "--no-mount", "home,cwd,hostfs,bind-paths", "--no-privs", "--drop-caps", "all"]
        if spec.gpu:
            a.append("--nv")
        if NetworkPolicy(spec.network) is NetworkPolicy.NONE:
            a += ["--net", "--network", "none"]
        a += ["--pwd", spec.workdir]
        for b in spec.binds:
            a += ["--bind", b.render()]
        for k, v in spec.env:
            a += ["--env", f"{k}={v}"]
        if spec.protected_output is not None:
            a += ["--env", f"{PROTECTED_OUTPUT_ENV}={spec.protected_output.sandbox_socket}"]
        a += [spec.image, self.shell, "-c", _in_container_script(spec)]
        return a

    def _payload_argv(self, spec: RunSpec) -> list:
        if not self.available():
            raise SandboxError(f"{self.bin} is not installed; use LocalSandbox for trusted payloads")
        return [self.bin] + self.build_argv(spec)


class LocalSandbox(_SupervisedSandbox):
    """No container: the payload runs as a child of the native supervisor with rlimits,
    wall clock, scratch cap and group kill, a scrubbed environment and its own cwd.
    For tests and trusted verifiers only."""

    @staticmethod
    def _host_path(spec: RunSpec, value: str) -> str:
        """Without a container a bind is only a name: a path beneath a bind's container side is
        rewritten to the same path beneath its host side (longest container prefix first)."""
        for b in sorted(spec.binds, key=lambda b: -len(b.container)):
            c = b.container.rstrip("/")
            if value == c or value.startswith(c + "/"):
                return b.host.rstrip("/") + value[len(c):]
        return value

    def _payload_argv(self, spec: RunSpec) -> list:
        import dataclasses
        wd = self._host_path(spec, spec.workdir)
        local = dataclasses.replace(spec, command=[self._host_path(spec, c) for c in spec.command])
        shell = "/bin/bash" if os.path.exists("/bin/bash") else "/bin/sh"      # `ulimit -u` is a bash spelling
        return [shell, "-c", f"cd {shell_quote(wd if os.path.isdir(wd) else '/')} && " + _in_container_script(local)]

    def _env(self, spec: RunSpec) -> dict:
        env = super()._env(spec)
        env.update({k: self._host_path(spec, v) for k, v in spec.env})
        if spec.protected_output is not None:
            env[PROTECTED_OUTPUT_ENV] = spec.protected_output.host_socket     # no container: host paths are the paths
        return env


class FakeSandbox(Sandbox):
    """Scripted double: ``fn(spec) -> SandboxOutcome``; records every spec it was given."""

    def __init__(self, fn: Callable[[RunSpec], SandboxOutcome]):
        self.fn = fn
        self.calls: list = []

    def run(self, spec: RunSpec) -> SandboxOutcome:
        self.calls.append(spec)
        return self.fn(spec)


def make_scratch(root: Optional[str] = None) -> str:
    return tempfile.mkdtemp(prefix="ferrl-scratch-", dir=root)
