import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
for p in (ROOT, ROOT / "oracle", ROOT / "tests"):
    if str(p) not in sys.path:
        sys.path.insert(0, str(p))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run with -m gpu on a B200)")


@pytest.fixture(scope="session")
def oracle():
    import oracle_lib
    oracle_lib.lib()
    return oracle_lib


@pytest.fixture(scope="session")
def ops():
    """The product ops; building/loading failures are test failures, never skips."""
    import torch
    assert torch.cuda.is_available(), "gpu-marked test collected without a CUDA device"
    from ds4cuda_b200 import ops as _ops, _lib
    _lib.load()
    return _ops


@pytest.fixture(scope="session")
def ref():
    """Reference kernels rebuilt for sm_100a (oracle/_ref/libds4ref.so).  The built library travels with
    the tree to the GPU box, so a GPU run without it means the build step failed: that is a test failure,
    not a skip (otherwise every bit-for-bit comparison with the reference would silently drop out)."""
    import ref_lib
    assert ref_lib.available(), (
        "oracle/_ref/libds4ref.so is missing: run `make -C oracle ref REF=<reference tree>` "
        "(__graft_entry__.build() does it when the reference tree is reachable)")
    return ref_lib
