"""The shipped examples run to completion."""
import os
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def _run(module, *args, timeout=180):
    env = dict(os.environ, PYTHONPATH=str(ROOT))
    return subprocess.run([sys.executable, "-m", module, *args], env=env, cwd=str(ROOT), capture_output=True, text=True,
                          timeout=timeout)


def test_pytorch_cpu_example():
    out = _run("execution_ucx_b200.axon.examples.pytorch_example")
    assert out.returncode == 0, out.stderr[-2000:]
    assert "result is the tensor the policy returned: True" in out.stdout
    assert "add_all: [[1.0, 1.0, 1.0], [2.0, 2.0, 2.0, 2.0, 2.0]]" in out.stdout


def test_jax_example_is_gated():
    out = _run("execution_ucx_b200.axon.examples.jax_example")
    assert out.returncode == 0, out.stderr[-2000:]


@pytest.mark.gpu
def test_pytorch_cuda_example(cuda_device):
    out = _run("execution_ucx_b200.axon.examples.pytorch_cuda_example")
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.count("same object as the policy's tensor: True") == 2
