import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on the B200 box)")


@pytest.fixture(scope="session")
def oracle_mod():
    """The CPU checker (oracle/), built on first use."""
    from oracle import build_oracle

    build_oracle.build_oracle()
    from oracle import oracle

    return oracle


@pytest.fixture(scope="session")
def cuda_lib():
    """The CUDA library behind the C ABI; GPU tests fail loudly if it is missing."""
    import torch

    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from hades_b200 import _lib

    lib = _lib.load()
    yield lib
    assert _lib.device_status() == 0, "a kernel recorded a device-side error"


GOLDEN = ROOT / "tests" / "golden"
