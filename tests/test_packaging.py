"""The wheel: built offline from the source tree, it carries the kernels' and the runtime's shared libraries
and the Python module, and a process that sees nothing but the installed wheel can make an RPC."""
import subprocess
import sys
import zipfile
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent


def test_wheel_builds_and_runs_from_a_clean_target(tmp_path):
    wh, inst = tmp_path / "wh", tmp_path / "inst"
    out = subprocess.run([sys.executable, "-m", "pip", "wheel", "--no-index", "--no-build-isolation", "--no-deps", "-w", str(wh), str(ROOT)],
                         capture_output=True, text=True, timeout=1500)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    wheels = list(wh.glob("execution_ucx_b200-*.whl"))
    assert len(wheels) == 1 and "linux" in wheels[0].name          # tagged for the platform: it carries machine code
    names = zipfile.ZipFile(wheels[0]).namelist()
    assert "execution_ucx_b200/_lib/libeux_kernels.so" in names and "execution_ucx_b200/_lib/libeux_runtime.so" in names
    assert any(n.startswith("execution_ucx_b200/axon/_axon") and n.endswith(".so") for n in names)
    assert "execution_ucx_b200/axon/examples/pytorch_example.py" in names
    out = subprocess.run([sys.executable, "-m", "pip", "install", "--no-index", "--no-deps", "--target", str(inst), str(wheels[0])],
                         capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stderr[-2000:]
    prog = (
        "import asyncio, numpy as np, execution_ucx_b200\n"
        "from execution_ucx_b200 import axon\n"
        "assert execution_ucx_b200.__file__.startswith(%r), execution_ucx_b200.__file__\n"
        "async def main():\n"
        "    s = axon.AxonRuntime('whl_server', timeout=5000); c = axon.AxonRuntime('whl_client', timeout=5000)\n"
        "    async def add(x: np.ndarray, k: int) -> np.ndarray:\n"
        "        return x + k\n"
        "    s.register_function(add); s.start_server(); c.start_client()\n"
        "    await c.connect_endpoint_async(s.get_local_address(), 'whl_server')\n"
        "    y = await c.invoke(np.arange(8, dtype=np.float32), 3, worker_name='whl_server', session_id=1, function='add', from_dlpack_fn=np.from_dlpack)\n"
        "    assert float(y[7]) == 10.0\n"
        "    c.stop(); s.stop()\n"
        "asyncio.run(main()); print('WHEEL_OK')\n" % str(inst))
    out = subprocess.run([sys.executable, "-c", prog], capture_output=True, text=True, timeout=300, cwd=str(tmp_path),
                         env={"PYTHONPATH": str(inst), "PATH": "/usr/bin:/bin"})
    assert out.returncode == 0 and "WHEEL_OK" in out.stdout, out.stdout[-1000:] + out.stderr[-3000:]
