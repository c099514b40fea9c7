"""In-tree build of the native library ``ferrl_b200/_C.so`` for sm_100a.

Every ``csrc/**/*.cu`` is compiled with ``nvcc -gencode arch=compute_100a,code=sm_100a``
(kernels include no torch headers, so each file takes seconds), ``csrc/*.cpp`` with
the host compiler against the torch headers, and everything is linked into one
shared object that ``ferrl_b200.ops.cuda`` loads with ``torch.ops.load_library``.
Objects are cached under ``build/`` keyed by a hash of source + flags, so a
second call is a no-op.  Cross-compiles without a GPU.
"""
from __future__ import annotations

import concurrent.futures as cf
import glob
import hashlib
import os
import shutil
import subprocess
import sys

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "csrc")
BUILD = os.path.join(ROOT, "build")
SO_PATH = os.path.join(ROOT, "ferrl_b200", "_C.so")
LAUNCHER_SRC = os.path.join(CSRC, "native", "sandbox_launcher.cpp")
LAUNCHER_BIN = os.path.join(ROOT, "ferrl_b200", "bin", "ferrl-sandbox-launch")

IO_SRC = os.path.join(CSRC, "native", "st_reader.cpp")
IO_LIB = os.path.join(ROOT, "ferrl_b200", "bin", "libferrl_io.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "--use_fast_math", "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr"]


def _nvcc() -> str:
    for cand in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if cand and os.path.exists(cand):
            return cand
    raise RuntimeError("nvcc not found")


def _hash(paths, extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode() + b"\0" + f.read())
    return h.hexdigest()[:16]


def _run(cmd, log_path=None):
    res = subprocess.run(cmd, capture_output=True, text=True)
    if log_path:
        with open(log_path, "w") as f:
            f.write(" ".join(cmd) + "\n" + res.stdout + res.stderr)
    if res.returncode != 0:
        raise RuntimeError(f"build step failed: {' '.join(cmd)}\n{res.stdout}\n{res.stderr}")
    return res


def build_launcher(force: bool = False) -> str:
    """Standalone host binary (no CUDA, no torch): the sandbox supervisor."""
    os.makedirs(os.path.dirname(LAUNCHER_BIN), exist_ok=True)
    if force or not os.path.exists(LAUNCHER_BIN) or os.path.getmtime(LAUNCHER_BIN) < os.path.getmtime(LAUNCHER_SRC):
        _run(["g++", "-O2", "-std=c++17", "-o", LAUNCHER_BIN, LAUNCHER_SRC])
    return LAUNCHER_BIN


def build_io(force: bool = False) -> str:
    """Host-only shared library (no CUDA, no torch): the safetensors range reader."""
    os.makedirs(os.path.dirname(IO_LIB), exist_ok=True)
    if force or not os.path.exists(IO_LIB) or os.path.getmtime(IO_LIB) < os.path.getmtime(IO_SRC):
        _run(["g++", "-O2", "-std=c++17", "-shared", "-fPIC", "-pthread", "-o", IO_LIB, IO_SRC])
    return IO_LIB


def build(force: bool = False, verbose: bool = False) -> str:
    import torch
    from torch.utils import cpp_extension as ce
    os.makedirs(BUILD, exist_ok=True)
    headers = glob.glob(os.path.join(CSRC, "**", "*.h"), recursive=True) + \
        glob.glob(os.path.join(CSRC, "**", "*.cuh"), recursive=True)
    cu = sorted(glob.glob(os.path.join(CSRC, "**", "*.cu"), recursive=True))
    cpp = sorted(p for p in glob.glob(os.path.join(CSRC, "**", "*.cpp"), recursive=True)
                 if os.sep + "native" + os.sep not in p)   # csrc/native holds standalone host programs
    build_launcher(force)
    build_io(force)
    nvcc = _nvcc()
    cuda_home = os.path.dirname(os.path.dirname(nvcc))
    inc = [f"-I{p}" for p in ce.include_paths()] + [f"-I{os.path.join(cuda_home, 'include')}"]
    abi = int(getattr(torch._C, "_GLIBCXX_USE_CXX11_ABI", True))
    jobs = []
    objs = []
    for src in cu:
        key = _hash([src] + headers, " ".join(NVCC_FLAGS))
        obj = os.path.join(BUILD, os.path.basename(src) + f".{key}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append(([nvcc] + NVCC_FLAGS + ["-c", src, "-o", obj], obj + ".log"))
    cxx_flags = ["-O2", "-std=c++17", "-fPIC", f"-D_GLIBCXX_USE_CXX11_ABI={abi}", "-DTORCH_API_INCLUDE_EXTENSION_H"]
    for src in cpp:
        key = _hash([src] + headers, " ".join(cxx_flags) + torch.__version__)
        obj = os.path.join(BUILD, os.path.basename(src) + f".{key}.o")
        objs.append(obj)
        if force or not os.path.exists(obj):
            jobs.append((["g++"] + cxx_flags + inc + ["-c", src, "-o", obj], obj + ".log"))
    if jobs:
        with cf.ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            for fut in [ex.submit(_run, c, l) for c, l in jobs]:
                res = fut.result()
                if verbose:
                    sys.stderr.write(res.stderr)
    stamp = os.path.join(BUILD, "link.stamp")
    want = _hash(objs, "link")
    have = open(stamp).read() if os.path.exists(stamp) else ""
    if force or jobs or have != want or not os.path.exists(SO_PATH):
        libdirs = ce.library_paths(device_type="cuda")
        link = ["g++", "-shared", "-o", SO_PATH] + objs + [f"-L{d}" for d in libdirs] + \
            [f"-Wl,-rpath,{d}" for d in libdirs] + \
            ["-lc10", "-ltorch_cpu", "-ltorch", "-lc10_cuda", "-ltorch_cuda", "-lcudart"]
        _run(link)
        with open(stamp, "w") as f:
            f.write(want)
    keep = {os.path.basename(o) for o in objs}
    for name in os.listdir(BUILD):   # objects of earlier source versions
        base = name[:-4] if name.endswith(".log") else name
        if base.endswith(".o") and base not in keep:
            os.remove(os.path.join(BUILD, name))
    return SO_PATH


if __name__ == "__main__":
    print(build(force="--force" in sys.argv, verbose=True))
