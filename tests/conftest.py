import os
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))


def pytest_configure(config):
    config.addinivalue_line("markers", "gpu: needs a CUDA device (run on a B200)")


@pytest.fixture(scope="session")
def native_build():
    """Build every native target once per session (no-op when up to date)."""
    from execution_ucx_b200 import _build
    _build.build_all()
    return _build


@pytest.fixture(scope="session")
def cuda_device():
    import torch
    if not torch.cuda.is_available():
        pytest.skip("no CUDA device")
    from execution_ucx_b200.ops import _native
    _native.load()  # fail loudly if the kernels library is missing on a GPU box
    return torch.device("cuda", 0)
