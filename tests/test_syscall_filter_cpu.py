"""The payload's seccomp policy: verdicts of the assembled filter on hand-made syscall records, and the
installed filter's effect in a child process.  Reference policy: crates/ferrl/src/trimul_eval_driver.py:267-375."""
import errno
import os
import platform
import socket
import subprocess
import sys
import textwrap

import pytest

from ferrl_b200.rewards.trimul_eval import syscall_filter as F

EPERM = F.RET_ERRNO | errno.EPERM


def test_filter_verdicts():
    prog = F.build_policy()
    assert all(0 <= jt <= 255 and 0 <= jf <= 255 for _, jt, jf, _ in prog)
    run = lambda nr, **kw: F.evaluate(prog, nr, **kw)   # noqa: E731
    assert run(0) == F.RET_ALLOW and run(1) == F.RET_ALLOW and run(9) == F.RET_ALLOW           # read, write, mmap
    assert run(0, arch=0x40000003) == F.RET_KILL_PROCESS                                        # i386 numbering
    assert run(F.X32_BIT | 1) == EPERM                                                          # x32 numbering
    for name in F.DENIED:
        assert run(F.SYSCALLS[name]) == EPERM, name
    assert run(F.SYSCALLS["clone3"]) == F.RET_ERRNO | errno.ENOSYS
    assert run(F.SYSCALLS["clone"], args=(0x00000011, 0, 0, 0, 0, 0)) == F.RET_ALLOW            # plain fork-style clone
    for flag in (0x00020000, 0x02000000, 0x04000000, 0x08000000, 0x10000000, 0x20000000, 0x40000000):
        assert run(F.SYSCALLS["clone"], args=(flag | 0x11, 0, 0, 0, 0, 0)) == EPERM             # every namespace flag
    for call in ("socket", "socketpair"):
        assert run(F.SYSCALLS[call], args=(socket.AF_UNIX, 1, 0, 0, 0, 0)) == F.RET_ALLOW
        for fam in (socket.AF_INET, socket.AF_INET6, 16, 17):                                    # netlink, packet
            assert run(F.SYSCALLS[call], args=(fam, 1, 0, 0, 0, 0)) == EPERM


def test_assembler_rejects_bad_programs():
    p = F.Program()
    p.jump_if_equal(1, then="nowhere")
    with pytest.raises(KeyError):
        p.assemble()
    p = F.Program()
    p.label("a")
    with pytest.raises(ValueError):
        p.label("a")


@pytest.mark.skipif(platform.machine() != "x86_64" or not sys.platform.startswith("linux"), reason="x86_64 Linux policy")
def test_installed_filter_in_a_child_process():
    code = textwrap.dedent("""
        import os, socket, sys, json
        sys.path.insert(0, %r)
        import syscall_filter as F
        try:
            ev = F.install()
        except OSError as e:
            print(json.dumps({"refused": str(e)})); sys.exit(0)
        out = {"ev": ev}
        try:
            socket.socket(socket.AF_INET, socket.SOCK_STREAM); out["inet"] = "allowed"
        except PermissionError:
            out["inet"] = "refused"
        a, b = socket.socketpair(); a.close(); b.close(); out["unix"] = "ok"
        pid = os.fork()
        if pid == 0:
            os._exit(7)
        out["child"] = os.waitpid(pid, 0)[1] >> 8
        try:
            os.unshare(0x20000000) if hasattr(os, "unshare") else (_ for _ in ()).throw(PermissionError())
            out["unshare"] = "allowed"
        except PermissionError:
            out["unshare"] = "refused"
        print(json.dumps(out))
    """) % os.path.dirname(F.__file__)
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=60)
    assert r.returncode == 0, r.stderr
    import json
    out = json.loads(r.stdout.strip().splitlines()[-1])
    if "refused" in out:
        pytest.skip("the kernel refused a seccomp filter here: " + out["refused"])
    assert out["ev"]["seccomp_mode"] == 2 and out["ev"]["no_new_privs"] == 1 and out["ev"]["seccomp_policy"] == F.POLICY_NAME
    assert out["inet"] == "refused" and out["unix"] == "ok" and out["child"] == 7 and out["unshare"] == "refused"
