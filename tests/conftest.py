import os
import sys

import pytest

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))   # tests dir: shared helpers such as _numerics

FIXTURES = os.path.join(os.path.dirname(os.path.abspath(__file__)), "fixtures")


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (sm_100a) and the built native extension")
    config.addinivalue_line("markers", "no_canary: run without canary-padded outputs (tests that measure allocator peaks)")


@pytest.fixture(scope="session")
def fixtures_dir():
    return FIXTURES


@pytest.fixture(autouse=True)
def _canary_padded_outputs(request):
    """Every GPU test runs with the native library's outputs allocated between pattern-filled pads; a kernel
    that stored outside one of its outputs fails the test here (tests that measure memory opt out with the
    ``no_canary`` marker)."""
    if request.node.get_closest_marker("gpu") is None or request.node.get_closest_marker("no_canary") is not None:
        yield
        return
    import torch
    if not torch.cuda.is_available():
        yield
        return
    from ferrl_b200.ops import cuda as C
    lib = C.lib()
    lib.set_canary(True)
    try:
        yield
        torch.cuda.synchronize()
        bad = lib.check_canaries()
    finally:
        lib.set_canary(False)
        lib.check_canaries()
    assert bad == 0, f"{bad} byte(s) written outside an output buffer"
