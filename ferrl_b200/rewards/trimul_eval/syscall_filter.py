"""Seccomp filter for the untrusted payload process of the TriMul evaluation.

The reference's in-sandbox driver installs a classic-BPF deny list before any candidate code runs
(crates/ferrl/src/trimul_eval_driver.py:267-375, policy name ``x86_64-tsync-af-unix-v1``): compute, file
and process syscalls that CUDA, PyTorch and compiler children need stay open, while cross-process
inspection, namespace and mount changes, kernel attack surfaces (bpf, io_uring, userfaultfd, perf, keyrings,
handle-based opens, pidfd access) and every socket family other than ``AF_UNIX`` are refused.  This module
builds a filter with the same policy from a small assembler with symbolic labels (no hand-counted jump
offsets), installs it on all threads of the calling process, and reports what the kernel says about the
result.  Stand-alone on purpose: the evaluation driver is copied into the sandbox as plain files and may
import nothing from the package.

Policy, in evaluation order:

1. a syscall from another architecture kills the process;
2. an x32 syscall (same audit architecture, different numbering) fails with ``EPERM``;
3. a denied syscall fails with ``EPERM``;
4. ``clone3`` fails with ``ENOSYS`` (its flags sit behind a pointer that a classic filter cannot read; libc
   falls back to ``clone``);
5. ``clone`` with any namespace flag fails with ``EPERM``;
6. ``socket`` / ``socketpair`` with a family other than ``AF_UNIX`` fail with ``EPERM``;
7. everything else is allowed.
"""
from __future__ import annotations

import ctypes
import errno
import os
import platform
import struct

POLICY_NAME = "x86_64-tsync-af-unix-v1"

# x86_64 syscall numbers (arch/x86/entry/syscalls/syscall_64.tbl)
SYSCALLS = {
    "socket": 41, "socketpair": 53, "clone": 56, "ptrace": 101, "pivot_root": 155, "chroot": 161, "mount": 165,
    "umount2": 166, "add_key": 248, "request_key": 249, "keyctl": 250, "unshare": 272, "perf_event_open": 298,
    "name_to_handle_at": 303, "open_by_handle_at": 304, "setns": 308, "process_vm_readv": 310,
    "process_vm_writev": 311, "kcmp": 312, "bpf": 321, "userfaultfd": 323, "pidfd_send_signal": 424,
    "io_uring_setup": 425, "io_uring_enter": 426, "io_uring_register": 427, "open_tree": 428, "move_mount": 429,
    "fsopen": 430, "fsconfig": 431, "fsmount": 432, "fspick": 433, "pidfd_open": 434, "clone3": 435,
    "pidfd_getfd": 438, "process_madvise": 440, "mount_setattr": 442, "process_mrelease": 448,
}
DENIED = ("ptrace", "pivot_root", "chroot", "mount", "umount2", "add_key", "request_key", "keyctl", "unshare",
          "perf_event_open", "name_to_handle_at", "open_by_handle_at", "setns", "process_vm_readv",
          "process_vm_writev", "kcmp", "bpf", "userfaultfd", "pidfd_send_signal", "io_uring_setup", "io_uring_enter",
          "io_uring_register", "open_tree", "move_mount", "fsopen", "fsconfig", "fsmount", "fspick", "pidfd_open",
          "pidfd_getfd", "process_madvise", "mount_setattr", "process_mrelease")

AUDIT_ARCH_X86_64 = 0xC000003E
X32_BIT = 0x40000000
CLONE_NAMESPACE_FLAGS = 0x7E020000      # CLONE_NEWNS | NEWCGROUP | NEWUTS | NEWIPC | NEWUSER | NEWPID | NEWNET
AF_UNIX = 1

RET_KILL_PROCESS = 0x80000000
RET_ERRNO = 0x00050000
RET_ALLOW = 0x7FFF0000

# offsets into struct seccomp_data {int nr; __u32 arch; __u64 ip; __u64 args[6];} (little endian: low words)
OFF_NR, OFF_ARCH, OFF_ARG0 = 0, 4, 16

_LD_ABS_W, _JEQ_K, _JSET_K, _RET_K = 0x20, 0x15, 0x45, 0x06


class Program:
    """Classic-BPF assembler: jumps name labels, ``assemble`` resolves them to forward offsets."""

    def __init__(self):
        self.ins = []           # (code, jt, jf, k) with jt/jf either None (fall through) or a label
        self.labels = {}

    def load(self, offset):
        self.ins.append((_LD_ABS_W, None, None, offset))

    def ret(self, value):
        self.ins.append((_RET_K, None, None, value))

    def jump_if_equal(self, value, then=None, otherwise=None):
        self.ins.append((_JEQ_K, then, otherwise, value))

    def jump_if_any_bit(self, mask, then=None, otherwise=None):
        self.ins.append((_JSET_K, then, otherwise, mask))

    def label(self, name):
        if name in self.labels:
            raise ValueError(f"label {name!r} defined twice")
        self.labels[name] = len(self.ins)

    def assemble(self):
        out = []
        for pc, (code, jt, jf, k) in enumerate(self.ins):
            def off(target):
                if target is None:
                    return 0
                d = self.labels[target] - (pc + 1)
                if not 0 <= d <= 255:
                    raise ValueError(f"jump to {target!r} out of range ({d})")
                return d
            out.append((code, off(jt), off(jf), k & 0xFFFFFFFF))
        if len(out) > 4096:
            raise ValueError("filter too long")
        return out


def build_policy() -> list:
    """The filter as a list of ``(code, jt, jf, k)`` tuples."""
    p = Program()
    eperm, enosys = RET_ERRNO | errno.EPERM, RET_ERRNO | errno.ENOSYS
    p.load(OFF_ARCH)
    p.jump_if_equal(AUDIT_ARCH_X86_64, then="arch_ok")
    p.ret(RET_KILL_PROCESS)
    p.label("arch_ok")
    p.load(OFF_NR)
    p.jump_if_any_bit(X32_BIT, otherwise="native_abi")
    p.ret(eperm)
    p.label("native_abi")
    for i, name in enumerate(DENIED):
        p.jump_if_equal(SYSCALLS[name], otherwise=f"not_{i}")
        p.ret(eperm)
        p.label(f"not_{i}")
    p.jump_if_equal(SYSCALLS["clone3"], otherwise="not_clone3")
    p.ret(enosys)
    p.label("not_clone3")
    p.jump_if_equal(SYSCALLS["clone"], otherwise="not_clone")
    p.load(OFF_ARG0)
    p.jump_if_any_bit(CLONE_NAMESPACE_FLAGS, otherwise="allow")
    p.ret(eperm)
    p.label("not_clone")
    p.jump_if_equal(SYSCALLS["socket"], then="family")
    p.jump_if_equal(SYSCALLS["socketpair"], otherwise="allow")
    p.label("family")
    p.load(OFF_ARG0)
    p.jump_if_equal(AF_UNIX, then="allow")
    p.ret(eperm)
    p.label("allow")
    p.ret(RET_ALLOW)
    return p.assemble()


def evaluate(program, nr, arch=AUDIT_ARCH_X86_64, args=(0, 0, 0, 0, 0, 0)) -> int:
    """Interpret ``program`` on one ``seccomp_data`` record (for tests: the filter's verdict without a kernel)."""
    data = struct.pack("<iIQ6Q", nr if nr < 2 ** 31 else nr - 2 ** 32, arch, 0, *args)
    acc, pc = 0, 0
    while True:
        code, jt, jf, k = program[pc]
        pc += 1
        if code == _LD_ABS_W:
            acc = struct.unpack_from("<I", data, k)[0]
        elif code == _RET_K:
            return k
        elif code == _JEQ_K:
            pc += jt if acc == k else jf
        elif code == _JSET_K:
            pc += jt if acc & k else jf
        else:
            raise ValueError(f"unsupported opcode {code:#x}")


class _SockFilter(ctypes.Structure):
    _fields_ = [("code", ctypes.c_ushort), ("jt", ctypes.c_ubyte), ("jf", ctypes.c_ubyte), ("k", ctypes.c_uint32)]


class _SockFprog(ctypes.Structure):
    _fields_ = [("len", ctypes.c_ushort), ("filter", ctypes.POINTER(_SockFilter))]


_PR_SET_NO_NEW_PRIVS = 38
_SYS_SECCOMP = 317
_SECCOMP_SET_MODE_FILTER = 1
_SECCOMP_FILTER_FLAG_TSYNC = 1


def install() -> dict:
    """Install the policy on every thread of this process (``no_new_privs`` first).  Returns the evidence
    record; raises ``OSError`` when the kernel refuses and ``RuntimeError`` off x86_64."""
    if platform.machine() != "x86_64":
        raise RuntimeError("the syscall filter is written for x86_64")
    prog = build_policy()
    arr = (_SockFilter * len(prog))(*[_SockFilter(c, jt, jf, k) for c, jt, jf, k in prog])
    fprog = _SockFprog(len(prog), arr)
    libc = ctypes.CDLL(None, use_errno=True)
    if libc.prctl(_PR_SET_NO_NEW_PRIVS, 1, 0, 0, 0) != 0:
        e = ctypes.get_errno()
        raise OSError(e, "prctl(PR_SET_NO_NEW_PRIVS): " + os.strerror(e))
    libc.syscall.restype = ctypes.c_long
    rc = libc.syscall(ctypes.c_long(_SYS_SECCOMP), ctypes.c_ulong(_SECCOMP_SET_MODE_FILTER),
                      ctypes.c_ulong(_SECCOMP_FILTER_FLAG_TSYNC), ctypes.byref(fprog))
    if rc != 0:
        e = ctypes.get_errno()
        raise OSError(e, "seccomp(SET_MODE_FILTER, TSYNC): " + os.strerror(e))
    return evidence()


def evidence() -> dict:
    """What the kernel reports about this process (``/proc/self/status``) next to the policy's name."""
    fields = {}
    try:
        with open("/proc/self/status", encoding="ascii") as f:
            for line in f:
                key, sep, value = line.partition(":")
                if sep and key in ("NoNewPrivs", "Seccomp", "Seccomp_filters"):
                    fields[key] = value.strip()
    except OSError:
        pass

    def num(key):
        try:
            return int(fields.get(key, ""))
        except ValueError:
            return None
    return {"seccomp_policy": POLICY_NAME, "seccomp_tsync": True, "arch": platform.machine(),
            "no_new_privs": num("NoNewPrivs"), "seccomp_mode": num("Seccomp"), "seccomp_filters": num("Seccomp_filters"),
            "instructions": len(build_policy())}
