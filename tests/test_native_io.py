"""Native safetensors range reader against the safetensors library."""
import json
import os
import struct

import pytest
import torch

from ferrl_b200.native import NativeIoError, SafetensorsFile
from ferrl_b200.models.loader import TensorSource


def _write(tmp_path, name="model.safetensors"):
    from safetensors.torch import save_file
    g = torch.Generator().manual_seed(3)
    tensors = {
        "a.weight": torch.randn(37, 24, generator=g).to(torch.bfloat16),
        "b.weight": torch.randn(64, 48, generator=g),
        "c.bias": torch.arange(19, dtype=torch.int64),
        "empty": torch.zeros(0, 8),
    }
    path = os.path.join(tmp_path, name)
    save_file(tensors, path, metadata={"format": "pt"})
    return path, tensors


def test_whole_rows_cols_match(tmp_path):
    path, tensors = _write(str(tmp_path))
    f = SafetensorsFile(path, threads=3, pin=False)
    assert sorted(f.keys()) == sorted(tensors)
    assert f.metadata == {"format": "pt"}
    for k, v in tensors.items():
        got = f.get(k)
        assert got.dtype == v.dtype and got.shape == v.shape and torch.equal(got, v)
    assert torch.equal(f.rows("a.weight", 5, 11), tensors["a.weight"][5:16])
    assert torch.equal(f.rows("c.bias", 18, 1), tensors["c.bias"][18:])
    assert torch.equal(f.cols("b.weight", 7, 30), tensors["b.weight"][:, 7:37])
    assert f.rows("a.weight", 3, 0).shape == (0, 24)
    with pytest.raises(IndexError):
        f.rows("a.weight", 30, 8)
    with pytest.raises(IndexError):
        f.cols("c.bias", 0, 1)


def test_large_range_uses_threads(tmp_path):
    from safetensors.torch import save_file
    w = torch.randn(3000, 1024)           # 12 MB: split over several positional reads
    path = os.path.join(str(tmp_path), "big.safetensors")
    save_file({"w": w}, path)
    f = SafetensorsFile(path, threads=4, pin=False)
    assert torch.equal(f.get("w"), w)
    assert torch.equal(f.cols("w", 100, 333), w[:, 100:433])


def test_bad_files_are_refused(tmp_path):
    p = os.path.join(str(tmp_path), "short.safetensors")
    with open(p, "wb") as fh:
        fh.write(struct.pack("<Q", 1 << 40))
    with pytest.raises(NativeIoError):
        SafetensorsFile(p, pin=False)
    with pytest.raises(NativeIoError):
        SafetensorsFile(os.path.join(str(tmp_path), "missing.safetensors"), pin=False)
    header = json.dumps({"w": {"dtype": "F32", "shape": [4, 4], "data_offsets": [0, 60]}}).encode()
    p2 = os.path.join(str(tmp_path), "lying.safetensors")
    with open(p2, "wb") as fh:
        fh.write(struct.pack("<Q", len(header)) + header + b"\0" * 64)
    with pytest.raises(ValueError):
        SafetensorsFile(p2, pin=False)


def test_tensor_source_native_equals_library(tmp_path):
    _, tensors = _write(str(tmp_path))
    nat, lib = TensorSource(str(tmp_path), native=True), TensorSource(str(tmp_path), native=False)
    assert type(nat._open["model.safetensors"]).__name__ == "SafetensorsFile"
    assert sorted(nat.names()) == sorted(lib.names())
    for k in ("a.weight", "b.weight"):
        assert torch.equal(nat.get(k), lib.get(k))
        assert torch.equal(nat.rows(k, 2, 9), lib.rows(k, 2, 9))
        assert torch.equal(nat.cols(k, 4, 10), lib.cols(k, 4, 10))
