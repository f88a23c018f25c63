"""A peer that goes away is detected on the host: the pending or next call fails with an error
(connection lost or deadline), nothing hangs, and the runtime keeps working with other peers.
The failure is made on the host side only (a process that exits between calls); no GPU is
faulted, and every device-side wait in the kernels has its own limit (see test_tensor_xfer_gpu)."""
import asyncio
import os
import subprocess
import sys
import time
from pathlib import Path

import pytest
import torch

ROOT = Path(__file__).resolve().parent.parent

SERVER = r"""
import asyncio, sys
import torch
from execution_ucx_b200 import axon

async def main(name, device):
    dev = None if device < 0 else axon.cuda(device)
    if device >= 0:
        torch.cuda.set_device(device)
    rt = axon.AxonRuntime(name, timeout=5000, device=dev)
    async def add_one(x: torch.Tensor) -> torch.Tensor:
        return x + 1.0
    pol = None
    if device >= 0:
        pol = lambda metas: torch.empty(metas[0].shape, dtype=torch.float32, device=f"cuda:{device}")
    rt.register_function(add_one, memory_policy=pol)
    rt.start_server()
    print("ADDRESS " + rt.get_local_address().hex(), flush=True)
    loop = asyncio.get_running_loop()
    line = await loop.run_in_executor(None, sys.stdin.readline)
    if line.strip() == "die":
        import os
        os._exit(3)          # no goodbye on the wire: the peer just disappears
    rt.stop()

asyncio.run(main(sys.argv[1], int(sys.argv[2])))
"""


def _spawn(tmp_path, name, device):
    script = tmp_path / "server.py"
    script.write_text(SERVER)
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    child = subprocess.Popen([sys.executable, str(script), name, str(device)], stdin=subprocess.PIPE, stdout=subprocess.PIPE,
                             env=env, cwd=str(ROOT))
    line = child.stdout.readline().decode().strip()
    assert line.startswith("ADDRESS "), line
    return child, bytes.fromhex(line.split()[1])


def _scenario(tmp_path, device):
    from execution_ucx_b200 import axon
    where = "cpu" if device < 0 else "cuda:0"
    first, addr1 = _spawn(tmp_path, "victim", device)
    second, addr2 = _spawn(tmp_path, "survivor", device)

    async def main():
        client = axon.AxonRuntime("fd_client", timeout=3000, device=None if device < 0 else axon.cuda(0))
        client.start_client()
        await client.connect_endpoint_async(addr1, "victim")
        await client.connect_endpoint_async(addr2, "survivor")
        pol = None if device < 0 else (lambda metas: torch.empty(metas[0].shape, dtype=torch.float32, device=where))
        x = torch.rand(50000, device=where)
        y = await client.invoke(x, worker_name="victim", session_id=1, function="add_one", memory_policy=pol)
        torch.testing.assert_close(y, x + 1.0)
        # the victim leaves between two calls, with nothing of ours in flight
        first.stdin.write(b"die\n")
        first.stdin.flush()
        first.wait(timeout=30)
        t0 = time.perf_counter()
        with pytest.raises(Exception) as err:
            await client.invoke(x, worker_name="victim", session_id=1, function="add_one", memory_policy=pol)
        took = time.perf_counter() - t0
        assert took < 10.0, f"the failure took {took:.1f} s to surface"
        text = str(err.value).lower()
        assert any(w in text for w in ("deadline", "unavailable", "connection", "closed", "reset", "not connected", "no endpoint")), text
        # the runtime is still good for the other peer
        y2 = await client.invoke(x, worker_name="survivor", session_id=2, function="add_one", memory_policy=pol)
        torch.testing.assert_close(y2, x + 1.0)
        client.stop()

    try:
        loop = asyncio.new_event_loop()
        loop.run_until_complete(main())
        loop.close()
    finally:
        for c in (first, second):
            if c.poll() is None:
                try:
                    c.stdin.write(b"quit\n")
                    c.stdin.flush()
                    c.wait(timeout=20)
                except Exception:
                    c.kill()


def test_peer_exit_is_detected_cpu(tmp_path):
    _scenario(tmp_path, -1)


@pytest.mark.gpu
@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_peer_exit_is_detected_two_gpus(tmp_path):
    _scenario(tmp_path, 1)
