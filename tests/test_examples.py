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


def test_foreign_array_example():
    """With JAX where it is installed, else with an array type that offers the DLPack protocol and nothing more."""
    out = _run("execution_ucx_b200.axon.examples.jax_example")
    assert out.returncode == 0, out.stderr[-2000:]
    assert "[0.0, 2.0, 4.0, 6.0, 8.0, 10.0, 12.0, 14.0]" in out.stdout, out.stdout


@pytest.mark.gpu
def test_pytorch_cuda_example(cuda_device):
    out = _run("execution_ucx_b200.axon.examples.pytorch_cuda_example")
    assert out.returncode == 0, out.stderr[-2000:]
    # the 4 KiB result arrives eagerly in the receive ring, the 64 MiB one in the tensor that the policy handed out
    assert out.stdout.count("received into the receive ring") == 1 and out.stdout.count("received into the policy's tensor") == 1, out.stdout


def test_text_trace_of_the_rpc_phases():
    """EUX_TRACE=1 writes the begin and end of every RPC phase to stderr, in the order a call goes through them."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), EUX_TRACE="1")
    out = subprocess.run([sys.executable, "-m", "execution_ucx_b200.axon.examples.pytorch_example"], env=env, cwd=str(ROOT),
                         capture_output=True, text=True, timeout=180)
    assert out.returncode == 0, out.stderr[-2000:]
    lines = [ln.split() for ln in out.stderr.splitlines() if ln.startswith("eux-trace ")]
    assert lines and all(len(ln) == 5 and ln[1] in ("B", "E", "M") and ln[3].isdigit() for ln in lines)
    lines.sort(key=lambda ln: int(ln[3]))  # several threads write: order by the clock, not by arrival
    names = [(ln[1], ln[2]) for ln in lines]
    # one call: the client starts it, the server dispatches it, the handler runs on the loop, the reply leaves
    # and the result is handed to the awaiting caller
    chain = [("B", "axon.client.invoke"), ("B", "axon.server.dispatch"), ("B", "axon.python.handler_on_loop"),
             ("B", "axon.server.send_response"), ("B", "axon.python.result_on_loop")]
    pos = 0
    for step in chain:
        assert step in names[pos:], (step, names[:40])
        pos = names.index(step, pos) + 1
    stamps = [int(ln[3]) for ln in lines]
    assert max(stamps) > min(stamps)
    assert sum(1 for k, _ in names if k == "B") == sum(1 for k, _ in names if k == "E")
