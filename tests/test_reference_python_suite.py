"""Runs the reference project's own Python test-suite against this package.

Set ``EUX_REFERENCE_PYTHON_TESTS`` to the directory that holds the reference's
``axon/python/tests`` (its ``test_*.py`` files and ``test_utils.py``). The suite is run
in a child pytest with ``execution_ucx_b200.axon`` importable as ``axon`` and coroutine
tests driven by ``execution_ucx_b200.axon.ref_suite_plugin``; every one of its cases has
to pass. Skipped when the variable is not set."""
import os
import re
import subprocess
import sys
from pathlib import Path

import pytest

ROOT = Path(__file__).resolve().parent.parent


def test_reference_python_suite_passes(tmp_path):
    suite = os.environ.get("EUX_REFERENCE_PYTHON_TESTS")
    if not suite:
        pytest.skip("EUX_REFERENCE_PYTHON_TESTS is not set")
    suite = str(Path(suite).resolve())
    env = dict(os.environ)
    env["PYTHONPATH"] = os.pathsep.join([str(ROOT), suite, env.get("PYTHONPATH", "")])
    # run from a scratch directory: the suite's folder is a package named `tests`, as this one is
    r = subprocess.run([sys.executable, "-m", "pytest", "-p", "execution_ucx_b200.axon.ref_suite_plugin", "-p", "no:cacheprovider",
                        "--import-mode=importlib", suite, "-q", "--timeout", "120"],
                       cwd=tmp_path, env=env, capture_output=True, text=True, timeout=1800)
    tail = r.stdout[-4000:] + r.stderr[-2000:]
    m = re.search(r"(\d+) passed", r.stdout)
    assert r.returncode == 0 and m, tail
    assert int(m.group(1)) >= 130, tail
