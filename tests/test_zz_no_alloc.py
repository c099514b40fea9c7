"""The allocation-free decode-attention entry point, called the way a host that cannot allocate
would call it: through the exported C symbol, with raw device pointers.

Such a host (a server that owns the whole device heap, a plugin running under someone else's
allocator lock) hands us its own input and output buffers and expects that the call itself
allocates nothing; the split-KV workspace is a fixed array inside the library.  The test checks
the result against the regular op - which takes its workspace from torch - on two consecutive
calls with different inputs, because the static array is shared and keeps the previous call's
contents, and checks that an oversized request is refused rather than overrunning the array.

This file sorts last on purpose, so a run that stops at the first failure has already run
every other test.
"""
import ctypes
import math
import os

import pytest
import torch

pytestmark = pytest.mark.gpu
SO = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "ferrl_b200", "_C.so")


def _entry():
    from ferrl_b200.ops import cuda as C
    C.lib()  # loads the library (and torch's CUDA libraries it links against)
    dll = ctypes.CDLL(SO)
    fn = dll.ferrl_decode_attn_static_ws
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p] * 5 + [ctypes.c_int] * 4 + [ctypes.c_longlong] * 2 + [ctypes.c_float] + \
        [ctypes.c_int] * 2 + [ctypes.c_void_p]
    err = dll.ferrl_noalloc_strerror
    err.restype = ctypes.c_char_p
    err.argtypes = [ctypes.c_int]
    return fn, err


def test_static_workspace_entry_matches_regular_op_twice():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    from ferrl_b200.ops import cuda as C
    fn, err = _entry()
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    B, Smax, Hq, Hkv, D, splits = 6, 700, 16, 4, 128, 4
    scale = 1.0 / math.sqrt(D)
    stream = torch.cuda.current_stream().cuda_stream
    for call in range(2):
        g = torch.Generator(device=dev).manual_seed(10 + call)
        q = torch.randn(B, Hq, D, device=dev, generator=g).to(torch.bfloat16)
        kc = torch.randn(B, Smax, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
        vc = torch.randn(B, Smax, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
        lens = torch.tensor([700, 1, 333, 64, 512 - call, 90 + 7 * call], device=dev, dtype=torch.int32)
        out = torch.empty_like(q)
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated(dev)
        free_before = torch.cuda.mem_get_info(dev)[0]      # a raw cudaMalloc would show here, not in torch's counter
        rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), out.data_ptr(), B, Hq, Hkv, D,
                kc.stride(0), kc.stride(1), scale, 0, splits, stream)
        assert rc == 0, err(rc)
        torch.cuda.synchronize()
        assert torch.cuda.memory_allocated(dev) == before   # nothing came from torch's allocator
        if call == 1:   # the first call on a device may load kernel images lazily; the second must not move the heap
            assert torch.cuda.mem_get_info(dev)[0] == free_before
        ref = C.decode_attention(q, kc, vc, lens, scale=scale, n_splits=splits)
        # same kernels, same split boundaries: the tolerance is the one the other decode tests use
        rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
        assert rel < 2e-2, rel
        assert torch.equal(out, ref)


def test_static_workspace_entry_on_the_second_device_before_the_first():
    """Kernel attributes (shared-memory opt-in for head dim 256) and the workspace address are kept per
    device: the first call of the process goes to device 1 with head dim 256, then the same to device 0."""
    if not torch.cuda.is_available() or torch.cuda.device_count() < 2:
        pytest.skip("needs two CUDA devices")
    from ferrl_b200.ops import cuda as C
    fn, err = _entry()
    B, Smax, Hq, Hkv, D, splits = 4, 300, 8, 2, 256, 2
    scale = 1.0 / math.sqrt(D)
    for index in (1, 0):
        dev = torch.device("cuda", index)
        with torch.cuda.device(dev):
            g = torch.Generator(device=dev).manual_seed(3 + index)
            q = torch.randn(B, Hq, D, device=dev, generator=g).to(torch.bfloat16)
            kc = torch.randn(B, Smax, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
            vc = torch.randn(B, Smax, Hkv, D, device=dev, generator=g).to(torch.bfloat16)
            lens = torch.tensor([300, 7, 129, 64], device=dev, dtype=torch.int32)
            out = torch.empty_like(q)
            stream = torch.cuda.current_stream(dev).cuda_stream
            rc = fn(q.data_ptr(), kc.data_ptr(), vc.data_ptr(), lens.data_ptr(), out.data_ptr(), B, Hq, Hkv, D,
                    kc.stride(0), kc.stride(1), scale, 0, splits, stream)
            assert rc == 0, err(rc)
            torch.cuda.synchronize(dev)
            ref = C.decode_attention(q, kc, vc, lens, scale=scale, n_splits=splits)
            assert torch.equal(out, ref), index


def test_static_workspace_entry_rejects_oversize_and_bad_args():
    if not torch.cuda.is_available():
        pytest.skip("needs a CUDA device")
    fn, err = _entry()
    dev = torch.device("cuda", 0)
    t = torch.zeros(16, device=dev, dtype=torch.bfloat16)
    lens = torch.zeros(1, device=dev, dtype=torch.int32)
    # 4096 * 32 * 16 * 130 floats is far beyond the 4 Mi-float array: refused before any launch
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), lens.data_ptr(), t.data_ptr(), 4096, 32, 8, 128, 0, 1024, 1.0, 0, 16, None)
    assert rc == 1 and b"exceeds" in err(rc)
    rc = fn(None, t.data_ptr(), t.data_ptr(), lens.data_ptr(), t.data_ptr(), 1, 4, 4, 128, 0, 512, 1.0, 0, 2, None)
    assert rc == 2
    rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), lens.data_ptr(), t.data_ptr(), 1, 4, 4, 100, 0, 400, 1.0, 0, 2, None)
    assert rc == 2
    # overlapping tokens (tok_stride < Hkv*D), a negative sequence stride and a negative window are refused
    for seq_stride, tok_stride, window in ((0, 511, 0), (-1, 512, 0), (0, 512, -1)):
        rc = fn(t.data_ptr(), t.data_ptr(), t.data_ptr(), lens.data_ptr(), t.data_ptr(), 1, 4, 4, 128,
                seq_stride, tok_stride, 1.0, window, 2, None)
        assert rc == 2 and b"tok_stride" in err(rc)
    torch.cuda.synchronize()
