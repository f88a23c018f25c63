"""Axon RPC with CUDA tensors: both runtimes in one process on GPU 0 (device payloads go through the
transfer kernel, not through host memory), and a two-process, two-GPU run when two GPUs are present."""
import asyncio
import os
import subprocess
import sys
from pathlib import Path
from typing import List

import pytest
import torch

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parent.parent


def run(coro):
    loop = asyncio.new_event_loop()
    try:
        asyncio.set_event_loop(loop)
        return loop.run_until_complete(coro)
    finally:
        loop.close()


def test_cuda_tensor_echo_same_process(cuda_device):
    from execution_ucx_b200 import axon

    async def main():
        server = axon.AxonRuntime("gpu_server", timeout=10000, device=axon.cuda(0))
        client = axon.AxonRuntime("gpu_client", timeout=10000, device=axon.cuda(0))

        async def plus_one(x: torch.Tensor) -> torch.Tensor:
            return x + 1.0

        async def concat_sizes(xs: List[torch.Tensor], k: int) -> List[torch.Tensor]:
            return [x * k for x in xs]

        def on_device(metas):
            outs = [torch.empty(m.shape, dtype=torch.float32, device="cuda:0") for m in metas]
            return outs if len(outs) > 1 else outs[0]

        server.register_function(plus_one, memory_policy=on_device)
        server.register_function(concat_sizes, memory_policy=lambda metas: [torch.empty(m.shape, dtype=torch.float32, device="cuda:0") for m in metas])
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "gpu_server")
        made = []

        def client_policy(metas):
            t = torch.empty(metas[0].shape, dtype=torch.float32, device="cuda:0")
            made.append(t)
            return t

        for n in (64, 4096, 1 << 19, (1 << 24) + 3):
            x = torch.rand(n, device="cuda:0")
            y = await client.invoke(x, worker_name="gpu_server", session_id=1, function="plus_one", memory_policy=client_policy)
            assert y.is_cuda and y.shape == x.shape
            if n * 4 > 64 << 10:
                assert y is made[-1], "large device results land in the tensor the policy returned"
            else:
                assert not made, "small device results arrive eagerly in the receive ring; the policy is not asked"
            torch.testing.assert_close(y, x + 1.0, rtol=0, atol=0)
            del y
        cs, ss = client.transport_stats(), server.transport_stats()
        # 256 B and 16 KiB went out as eager device messages in both directions (no rendezvous), 2 MiB was
        # pulled by the receiver's kernel, 64 MiB pushed by the sender's; nothing went through host memory
        assert cs["device_eager_sent"] == 2 and ss["device_eager_recv"] == 2, (cs, ss)
        assert ss["device_eager_sent"] == 2 and cs["device_eager_recv"] == 2, (cs, ss)
        assert cs["device_pushes"] == 1 and ss["device_push_recv"] == 1 and ss["device_pushes"] == 1 and cs["device_push_recv"] == 1, (cs, ss)
        assert ss["device_pulls"] == 1 and cs["device_pulls"] == 1, (cs, ss)
        assert cs["device_staged"] == 0 and ss["device_staged"] == 0, (cs, ss)
        # more eager messages than the ring has slots, all in flight at once: the surplus takes the rendezvous
        xs = [torch.full((256,), float(i), device="cuda:0") for i in range(80)]
        ys = await asyncio.gather(*[client.invoke(x, worker_name="gpu_server", session_id=2, function="plus_one", memory_policy=client_policy)
                                    for x in xs])
        for i, y in enumerate(ys):
            assert float(y[0]) == i + 1.0 and float(y[-1]) == i + 1.0
        del ys
        # 2-D, non-contiguous input is packed before it is sent
        x2 = torch.rand(300, 70, device="cuda:0").t()
        y2 = await client.invoke(x2, worker_name="gpu_server", session_id=1, function="plus_one", memory_policy=client_policy)
        torch.testing.assert_close(y2, x2.contiguous() + 1.0, rtol=0, atol=0)
        # a list of tensors travels as one scatter-gather message
        xs = [torch.rand(1000, device="cuda:0"), torch.rand(70000, device="cuda:0"), torch.rand(8, device="cuda:0")]
        ys = await client.invoke(xs, 3, worker_name="gpu_server", session_id=1, function="concat_sizes",
                                 memory_policy=lambda metas: [torch.empty(m.shape, dtype=torch.float32, device="cuda:0") for m in metas])
        assert len(ys) == 3
        for a, b in zip(xs, ys):
            torch.testing.assert_close(b, a * 3, rtol=0, atol=0)
        # device tensor received into host memory when no policy is given (staged copy)
        z = await client.invoke(torch.rand(50000, device="cuda:0"), worker_name="gpu_server", session_id=1, function="plus_one")
        assert z.shape == (50000,)
        client.stop()
        server.stop()

    run(main())


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_processes_two_gpus():
    """Server on GPU 1 in a child process, client on GPU 0 here: the payloads cross NVLink by the transfer
    kernels (eager into the ring, pulled, pushed), signalled through the shared flag page."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    child = subprocess.Popen([sys.executable, "-m", "execution_ucx_b200.models.echo_server", "--device", "1", "--name", "peer"],
                             stdout=subprocess.PIPE, stdin=subprocess.PIPE, env=env, cwd=str(ROOT))
    try:
        line = child.stdout.readline().decode().strip()
        assert line.startswith("ADDRESS "), line
        address = bytes.fromhex(line.split()[1])
        from execution_ucx_b200 import axon

        async def main():
            client = axon.AxonRuntime("client0", timeout=20000, device=axon.cuda(0))
            client.start_client()
            await client.connect_endpoint_async(address, "peer")
            policy = lambda metas: torch.empty(metas[0].shape, dtype=torch.bfloat16, device="cuda:0")  # noqa: E731
            for n in (1024, 1 << 20, 1 << 24):      # 2 KiB: eager into the peer's ring; 2 MiB: pulled; 32 MiB: pushed
                x = torch.randn(n, device="cuda:0").to(torch.bfloat16)
                y = await client.invoke(x, worker_name="peer", session_id=1, function="echo", memory_policy=policy)
                assert y.device.index == 0 and torch.equal(y.view(torch.int16), x.view(torch.int16))
                del y
            st = client.transport_stats()
            assert st["device_eager_sent"] == 1 and st["device_eager_recv"] == 1, st
            assert st["device_pulls"] == 1 and st["device_pushes"] == 1 and st["device_push_recv"] == 1, st
            assert st["device_staged"] == 0, st
            client.stop()

        run(main())
    finally:
        try:
            child.stdin.write(b"quit\n")
            child.stdin.flush()
            child.wait(timeout=30)
        except Exception:
            child.kill()


def test_expandable_segment_tensors_cross_processes_on_the_device_paths():
    """Tensors from the tensor library's expandable segments (cuMemCreate allocations, which have no CUDA
    IPC handle) between two processes: eager, pulled and pushed, nothing staged through the host. Runs in
    processes of its own because the allocator reads its configuration once."""
    env = dict(os.environ, PYTHONPATH=str(ROOT), PYTORCH_CUDA_ALLOC_CONF="expandable_segments:True", NCCL_NVLS_ENABLE="0")
    out = subprocess.run([sys.executable, str(ROOT / "tests" / "mp_vmm_gpu.py")], env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout[-2000:] + out.stderr[-4000:]
