"""CUDA preflight: refuse to start on hardware this build cannot run on, with a
typed error instead of a failure at the first kernel launch.

The reference checks PTX-ISA / driver compatibility tables and guards the first
kernel (``crates/ferrl/src/cuda_compat.rs:55-87``).  This build ships sm_100a
code only, so the check is: a CUDA device with compute capability 10.x, a
driver at least as new as the toolkit the kernels were built with, the native
library present and loadable, and - for multi-GPU runs - peer access between
every pair of local GPUs.  ``translate_cuda_error`` turns the loader's and the
driver's usual messages for those conditions into the same typed errors
(``cuda_compat.rs``: ``translate_ptx_error``, ``check_driver_compat``).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional


class PreflightError(RuntimeError):
    def __init__(self, kind: str, msg: str):
        super().__init__(msg)
        self.kind = kind


@dataclass
class DeviceReport:
    name: str
    capability: tuple
    total_memory: int
    sm_count: int
    peer_ok: bool


def check_device(index: int = 0, *, need_peers: Optional[int] = None, probe=None) -> DeviceReport:
    """``probe`` lets tests supply a fake of the few torch.cuda calls used here."""
    if probe is None:
        import torch
        probe = torch.cuda
    if not probe.is_available():
        raise PreflightError("no_device", "no CUDA device is visible")
    if index >= probe.device_count():
        raise PreflightError("no_device", f"device {index} requested but only {probe.device_count()} visible")
    cap = tuple(probe.get_device_capability(index))
    props = probe.get_device_properties(index)
    if cap[0] != 10:
        raise PreflightError("wrong_arch", f"{props.name} has compute capability {cap[0]}.{cap[1]}; this build "
                                           "contains sm_100a kernels only (Blackwell B200 class required)")
    peer_ok = True
    if need_peers and need_peers > 1:
        if probe.device_count() < need_peers:
            raise PreflightError("no_device", f"{need_peers} GPUs requested, {probe.device_count()} visible")
        for a in range(need_peers):
            for b in range(need_peers):
                if a != b and not probe.can_device_access_peer(a, b):
                    peer_ok = False
        if not peer_ok:
            raise PreflightError("no_peer_access", "not every pair of local GPUs has peer access; the symmetric "
                                                   "heap needs NVLink/NVSwitch peer mappings")
    return DeviceReport(props.name, cap, props.total_memory, props.multi_processor_count, peer_ok)


BUILT_WITH_CUDA = (12, 9)       # toolkit the in-tree kernels are compiled with


def check_driver_compat(driver_version: Optional[int], built_with: tuple = BUILT_WITH_CUDA) -> tuple:
    """``driver_version`` as the driver API reports it (``12090`` = 12.9).  sm_100a machine code
    needs no JIT, but the runtime the extension links refuses a driver older than its own major
    version, and a driver older than the toolkit's minor version cannot load newer-ISA PTX."""
    if not driver_version:
        raise PreflightError("no_driver", "the CUDA driver version could not be read (no driver loaded?)")
    major, minor = driver_version // 1000, (driver_version % 1000) // 10
    if (major, minor) < built_with:
        raise PreflightError("driver_too_old", f"the CUDA driver supports up to CUDA {major}.{minor}, but the kernels "
                                               f"were built with CUDA {built_with[0]}.{built_with[1]}; "
                                               "update the driver (or install the matching compat package)")
    return major, minor


_ERROR_HINTS = (
    ("no kernel image is available", "wrong_arch",
     "the binary holds sm_100a code only and this GPU is not a compute-capability-10.0 device"),
    ("invalid device function", "wrong_arch",
     "the binary holds sm_100a code only and this GPU is not a compute-capability-10.0 device"),
    ("unsupported toolchain", "driver_too_old",
     "the driver is older than the toolkit the kernels were built with"),
    ("unsupported ptx version", "driver_too_old",
     "the driver is older than the toolkit the kernels were built with"),
    ("driver version is insufficient", "driver_too_old",
     "the driver is older than the CUDA runtime this build links"),
    ("peer access is not supported", "no_peer_access",
     "the symmetric heap needs NVLink/NVSwitch peer mappings between the local GPUs"),
    ("out of memory", "out_of_memory", "the device ran out of memory"),
)


def translate_cuda_error(message: str) -> Optional[PreflightError]:
    """A typed error for the launch-time messages whose cause is the installation, else ``None``."""
    low = message.lower()
    for needle, kind, hint in _ERROR_HINTS:
        if needle in low:
            return PreflightError(kind, f"{hint} (driver said: {message.strip()[:200]})")
    return None


def guard_first_kernel() -> None:
    """Load the native library and run one trivial kernel so that a broken
    install surfaces here, with context, rather than deep inside a rollout."""
    import torch
    from .ops import ExtensionMissing, cuda as C
    try:
        lib = C.lib()
        x = torch.ones(8, 64, device="cuda", dtype=torch.bfloat16)
        y, _ = lib.rmsnorm(x, None, None, None, 1e-6, False)
        torch.cuda.synchronize()
    except ExtensionMissing:
        raise
    except RuntimeError as e:
        typed = translate_cuda_error(str(e))
        if typed is not None:
            raise typed from e
        raise PreflightError("first_kernel", f"the first kernel launch failed: {e}") from e
    if not bool(torch.isfinite(y.float()).all()):
        raise PreflightError("first_kernel", "the first kernel produced non-finite output")
