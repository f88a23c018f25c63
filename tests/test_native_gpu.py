"""The C++ tests that need a GPU: ucx_am_context with device memory (csrc/tests/am_context_cuda_test.cpp)."""
import subprocess
from pathlib import Path

import pytest

pytestmark = pytest.mark.gpu
LIB = Path(__file__).resolve().parent.parent / "execution_ucx_b200" / "_lib"


@pytest.mark.parametrize("binary", ["eux_am_context_cuda_test"])
def test_native_gpu_binary(binary, native_build, cuda_device):
    exe = LIB / binary
    assert exe.exists(), f"{exe} is not built: run python -m execution_ucx_b200._build"
    out = subprocess.run([str(exe)], capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-4000:] + out.stderr[-2000:]
    assert "0 failed" in out.stdout
