"""Host-side native helpers: the safetensors range reader.

``SafetensorsFile`` parses a shard's header and reads whole tensors, row ranges or
column ranges with threaded positional reads from ``libferrl_io.so``
(``csrc/native/st_reader.cpp``) straight into a (by default pinned, when CUDA is
present) host tensor, so a tensor-parallel rank touches only the bytes of its own
slice and the host->device copy can run asynchronously.

Reference behaviour: ``crates/ferrl/src/sharded_safetensors.rs:644-750`` (rank-local
streaming: seek to the byte range of this rank's rows/columns of every tensor) and the
header validation at ``:120-260`` (offsets contiguous, inside the file, dtype sizes
consistent with the shape).
"""
from __future__ import annotations

import ctypes
import json
import os
from typing import Optional

import torch

from . import _build

_DTYPES = {
    "F64": torch.float64, "F32": torch.float32, "F16": torch.float16, "BF16": torch.bfloat16,
    "I64": torch.int64, "I32": torch.int32, "I16": torch.int16, "I8": torch.int8, "U8": torch.uint8,
    "BOOL": torch.bool,
}
for _name, _attr in (("F8_E4M3", "float8_e4m3fn"), ("F8_E5M2", "float8_e5m2")):
    if hasattr(torch, _attr):
        _DTYPES[_name] = getattr(torch, _attr)

_lib = None


class NativeIoError(OSError):
    pass


def io_lib():
    """The loaded range-reader library (built on first use)."""
    global _lib
    if _lib is None:
        path = _build.IO_LIB if os.path.exists(_build.IO_LIB) else _build.build_io()
        lib = ctypes.CDLL(path)
        lib.ferrl_read_range.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int]
        lib.ferrl_read_range.restype = ctypes.c_int
        lib.ferrl_read_strided.argtypes = [ctypes.c_char_p, ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint64,
                                           ctypes.c_uint64, ctypes.c_void_p, ctypes.c_int]
        lib.ferrl_read_strided.restype = ctypes.c_int
        lib.ferrl_read_header.argtypes = [ctypes.c_char_p, ctypes.POINTER(ctypes.c_uint64), ctypes.c_char_p, ctypes.c_uint64]
        lib.ferrl_read_header.restype = ctypes.c_int
        _lib = lib
    return _lib


def _check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeIoError(-rc, f"{what}: {os.strerror(-rc)}")


class SafetensorsFile:
    """One ``.safetensors`` shard opened for range reads."""

    def __init__(self, path: str, threads: int = 0, pin: Optional[bool] = None):
        self.path = path
        self._cpath = os.fsencode(path)
        self.threads = threads
        self.pin = torch.cuda.is_available() if pin is None else pin
        lib = io_lib()
        n = ctypes.c_uint64(0)
        _check(lib.ferrl_read_header(self._cpath, ctypes.byref(n), None, 0), f"header of {path}")
        buf = ctypes.create_string_buffer(n.value)
        _check(lib.ferrl_read_header(self._cpath, ctypes.byref(n), buf, n.value), f"header of {path}")
        meta = json.loads(buf.raw[:n.value].decode("utf-8"))
        self.metadata = meta.pop("__metadata__", {})
        self.data_start = 8 + n.value
        size = os.path.getsize(path)
        self.entries: dict[str, tuple[torch.dtype, tuple[int, ...], int, int]] = {}
        for name, e in meta.items():
            if e["dtype"] not in _DTYPES:
                raise ValueError(f"{path}: tensor {name!r} has unsupported dtype {e['dtype']}")
            dt = _DTYPES[e["dtype"]]
            shape = tuple(int(d) for d in e["shape"])
            lo, hi = (int(v) for v in e["data_offsets"])
            numel = 1
            for d in shape:
                numel *= d
            if hi - lo != numel * dt.itemsize or lo < 0 or self.data_start + hi > size:
                raise ValueError(f"{path}: tensor {name!r} has inconsistent offsets {lo}..{hi} for shape {shape}")
            self.entries[name] = (dt, shape, self.data_start + lo, hi - lo)

    def keys(self):
        return list(self.entries.keys())

    def shape(self, name: str) -> tuple[int, ...]:
        return self.entries[name][1]

    def _empty(self, shape, dtype) -> torch.Tensor:
        return torch.empty(shape, dtype=dtype, pin_memory=self.pin)

    def get(self, name: str) -> torch.Tensor:
        dt, shape, off, nbytes = self.entries[name]
        out = self._empty(shape, dt)
        if nbytes:
            _check(io_lib().ferrl_read_range(self._cpath, off, nbytes, out.data_ptr(), self.threads), f"read {name}")
        return out

    def rows(self, name: str, start: int, n: int) -> torch.Tensor:
        """Rows ``[start, start+n)`` of the leading dimension (one contiguous byte range)."""
        dt, shape, off, _ = self.entries[name]
        if not shape or start < 0 or n < 0 or start + n > shape[0]:
            raise IndexError(f"rows {start}..{start + n} outside {name} with shape {shape}")
        row_bytes = dt.itemsize
        for d in shape[1:]:
            row_bytes *= d
        out = self._empty((n,) + shape[1:], dt)
        if n and row_bytes:
            _check(io_lib().ferrl_read_range(self._cpath, off + start * row_bytes, n * row_bytes, out.data_ptr(),
                                             self.threads), f"read rows of {name}")
        return out

    def cols(self, name: str, start: int, n: int) -> torch.Tensor:
        """Columns ``[start, start+n)`` of a matrix (one short read per row)."""
        dt, shape, off, _ = self.entries[name]
        if len(shape) != 2 or start < 0 or n < 0 or start + n > shape[1]:
            raise IndexError(f"cols {start}..{start + n} outside {name} with shape {shape}")
        out = self._empty((shape[0], n), dt)
        if n and shape[0]:
            _check(io_lib().ferrl_read_strided(self._cpath, off + start * dt.itemsize, shape[1] * dt.itemsize, shape[0],
                                               n * dt.itemsize, out.data_ptr(), self.threads), f"read cols of {name}")
        return out
