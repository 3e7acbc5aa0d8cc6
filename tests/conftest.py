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
    """Reference kernels rebuilt for sm_100a (oracle/_ref); None when not built."""
    import ref_lib
    return ref_lib if ref_lib.available() else None
