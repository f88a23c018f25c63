"""Runs the C++ unit-test binaries (built in-tree) that need no GPU."""
import subprocess
from pathlib import Path

import pytest

LIB = Path(__file__).resolve().parent.parent / "execution_ucx_b200" / "_lib"
BINARIES = ["eux_exec_test", "eux_transport_test", "eux_rpc_cases_test", "eux_cancel_test", "eux_am_context_test", "eux_data_test", "eux_rpc_test", "eux_axon_test", "eux_axon_typed_test", "eux_storage_test"]


@pytest.mark.parametrize("name", BINARIES)
def test_cpp_binary(native_build, name):
    exe = LIB / name
    if not exe.exists():
        src = Path(__file__).resolve().parent.parent / "csrc" / "tests" / (name[4:] + ".cpp")
        if not src.exists():
            pytest.skip(f"{name} has no source yet")
        pytest.fail(f"{exe} was not built")
    r = subprocess.run([str(exe)], capture_output=True, text=True, timeout=300)
    tail = "\n".join((r.stdout + r.stderr).splitlines()[-30:])
    assert r.returncode == 0, tail
