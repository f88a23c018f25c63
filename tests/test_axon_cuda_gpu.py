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
            if n * 4 > 16 << 20:
                assert y is made[-1], "large device results land in the tensor the policy returned"
            else:
                assert not made, "device results up to 16 MiB arrive eagerly in the receive ring; the policy is not asked"
            torch.testing.assert_close(y, x + 1.0, rtol=0, atol=0)
            del y
        cs, ss = client.transport_stats(), server.transport_stats()
        # 256 B, 16 KiB and 2 MiB went out as eager device messages in both directions (no rendezvous), 64 MiB
        # was pushed by the sender's kernel; nothing went through host memory
        assert cs["device_eager_sent"] == 3 and ss["device_eager_recv"] == 3, (cs, ss)
        assert ss["device_eager_sent"] == 3 and cs["device_eager_recv"] == 3, (cs, ss)
        assert cs["device_pushes"] == 1 and ss["device_push_recv"] == 1 and ss["device_pushes"] == 1 and cs["device_push_recv"] == 1, (cs, ss)
        assert ss["device_pulls"] == 0 and cs["device_pulls"] == 0, (cs, ss)
        assert cs["device_staged"] == 0 and ss["device_staged"] == 0, (cs, ss)
        # more eager messages than the ring has slots, all in flight at once: the surplus takes the rendezvous
        # and is pulled by the receiver's kernel
        xs = [torch.full((256,), float(i), device="cuda:0") for i in range(80)]
        ys = await asyncio.gather(*[client.invoke(x, worker_name="gpu_server", session_id=2, function="plus_one", memory_policy=client_policy)
                                    for x in xs])
        for i, y in enumerate(ys):
            assert float(y[0]) == i + 1.0 and float(y[-1]) == i + 1.0
        del ys
        assert client.transport_stats()["device_pulls"] + server.transport_stats()["device_pulls"] >= 1
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
            for n in (1024, 1 << 20, 1 << 24):      # 2 KiB, 2 MiB: eager into the peer's ring (one slot, two slots); 32 MiB: pushed
                x = torch.randn(n, device="cuda:0").to(torch.bfloat16)
                y = await client.invoke(x, worker_name="peer", session_id=1, function="echo", memory_policy=policy)
                assert y.device.index == 0 and torch.equal(y.view(torch.int16), x.view(torch.int16))
                del y
            st = client.transport_stats()
            assert st["device_eager_sent"] == 2 and st["device_eager_recv"] == 2, st
            assert st["device_pulls"] == 0 and st["device_pushes"] == 1 and st["device_push_recv"] == 1, st
            assert st["device_staged"] == 0, st
            # strided views cross NVLink as they lie: up to the eager limit gathered into the peer's ring by this
            # process's kernel (12 KiB, 2.7 MiB), a large one (32 MiB) gathered out of this process's memory by the peer's pull
            base = torch.randn(4096, 4096, device="cuda:0").to(torch.bfloat16)
            for view in (base[:64, :96].t(), base.t(), base[:2048:2, 1::3]):
                assert not view.is_contiguous()
                y = await client.invoke(view, worker_name="peer", session_id=1, function="echo", memory_policy=policy)
                assert y.shape == view.shape and torch.equal(y.view(torch.int16), view.contiguous().view(torch.int16))
                del y
            st2 = client.transport_stats()
            assert st2["device_gathers"] == 2 and st2["device_packs"] == 0 and st2["device_staged"] == 0, st2
            assert st2["device_push_recv"] == 2, st2     # the answer to the 32 MiB view is dense: the peer pushed it
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
    # the eager limit is set to 64 KiB so that the 2 MiB and 3 MiB payloads are pulled out of the sender's
    # segments by the receiver's kernel (by default they would be stored into the receiver's ring by the sender's)
    env = dict(os.environ, PYTHONPATH=str(ROOT), PYTORCH_CUDA_ALLOC_CONF="expandable_segments:True", NCCL_NVLS_ENABLE="0",
               EUX_DEV_EAGER_LIMIT="65536")
    out = subprocess.run([sys.executable, str(ROOT / "tests" / "mp_vmm_gpu.py")], env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=300)
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout[-2000:] + out.stderr[-4000:]


def test_strided_and_unfinished_tensors(cuda_device):
    """A strided view is sent as it lies (gathered by the transfer kernel: no dense copy is made first), and a
    tensor whose producer is still running is sent without waiting for it on the host: the result is that of
    the finished producer all the same."""
    from execution_ucx_b200 import axon

    async def main():
        server = axon.AxonRuntime("sg_server", timeout=20000, device=axon.cuda(0))
        client = axon.AxonRuntime("sg_client", timeout=20000, device=axon.cuda(0))
        table = {(2, 32): torch.float32, (2, 64): torch.float64, (4, 16): torch.bfloat16, (1, 8): torch.uint8, (0, 64): torch.int64}

        def on_device(metas):
            m = metas[0]
            return torch.empty(m.shape, dtype=table[(m.dtype.code, m.dtype.bits)], device="cuda:0")

        async def echo(x: torch.Tensor) -> torch.Tensor:
            return x

        server.register_function(echo, memory_policy=on_device)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "sg_server")
        big = torch.rand(1 << 24, device="cuda:0")
        views = [
            torch.rand(64, 50, device="cuda:0").t(),                         # 12.5 KiB: gathered into the ring slot
            torch.rand(300, 70, device="cuda:0").t(),                        # 82 KiB: the same, by a launch of several CTAs
            torch.rand(1200, 700, device="cuda:0").t(),                      # 3.2 MiB: gathered into a run of four slots
            big[::2],                                                        # 32 MiB, every other element
            big.view(256, 256, 256).permute(2, 0, 1),                        # 64 MiB, three dimensions
            torch.rand(40, 30, device="cuda:0", dtype=torch.float64).t(),    # 8-byte elements
            torch.arange(100, device="cuda:0").expand(50, 100),              # a stride of zero, int64
            torch.randint(0, 255, (70, 33), device="cuda:0", dtype=torch.uint8)[:, 1:],   # single bytes, odd offset
            torch.randn(128, 96, device="cuda:0").to(torch.bfloat16)[:, ::3],
        ]
        for v in views:
            assert not v.is_contiguous()
            y = await client.invoke(v, worker_name="sg_server", session_id=1, function="echo", memory_policy=on_device)
            assert y.shape == v.shape and y.dtype == v.dtype and y.is_contiguous()
            assert torch.equal(y, v.contiguous()), (v.shape, v.stride(), v.dtype)
            del y
        cs = client.transport_stats()
        # every view was gathered by a transfer (the echo's answers are dense): none was packed first
        assert cs["device_gathers"] + server.transport_stats()["device_gathers"] == len(views), (cs, server.transport_stats())
        assert cs["device_packs"] == 0 and cs["device_staged"] == 0, cs
        # a producer that is still running when the tensor is sent: ~50 ms of spinning, then the values
        side = torch.cuda.Stream(device="cuda:0")
        for n in (1 << 10, 1 << 22):                 # a small and a large one: either is announced once its producer is done
            x = torch.zeros(n, device="cuda:0")
            torch.cuda.synchronize()
            with torch.cuda.stream(side):
                torch.cuda._sleep(100_000_000)
                x.add_(7.0)
                fut = client.invoke(x, worker_name="sg_server", session_id=2, function="echo", memory_policy=on_device)
                assert not side.query(), "the send was issued while the producer was still running"
            y = await fut
            assert float(y.min()) == 7.0 and float(y.max()) == 7.0
            del y
        assert client.transport_stats()["sends_held"] >= 1
        client.stop()
        server.stop()

    run(main())


def test_tensors_converted_on_the_way(cuda_device):
    """``wire_dtype``: fp32 tensors travel as bf16 (or fp16), converted by the transfer kernel while it moves
    them: into the ring slot for a small one, by the receiver's pull for a large or a strided one. What arrives
    is the tensor rounded once to the wire type, and the function's fp32 result can come back the same way."""
    from execution_ucx_b200 import axon

    async def main():
        server = axon.AxonRuntime("cv_server", timeout=20000, device=axon.cuda(0))
        client = axon.AxonRuntime("cv_client", timeout=20000, device=axon.cuda(0))
        table = {(2, 32): torch.float32, (2, 16): torch.float16, (4, 16): torch.bfloat16}
        seen = []

        def on_device(metas):
            m = metas[0]
            return torch.empty(m.shape, dtype=table[(m.dtype.code, m.dtype.bits)], device="cuda:0")

        async def what_arrived(x: torch.Tensor) -> torch.Tensor:
            seen.append((x.dtype, tuple(x.shape)))
            return x

        async def as_fp32(x: torch.Tensor) -> torch.Tensor:
            return x.float() * 2.0

        server.register_function(what_arrived, memory_policy=on_device)
        server.register_function(as_fp32, memory_policy=on_device, wire_dtype=torch.bfloat16)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "cv_server")
        cases = [
            (torch.randn(1000, device="cuda:0"), torch.bfloat16),                       # 2 KiB on the wire: eager, converted on its way into the ring slot
            (torch.randn(1 << 20, device="cuda:0"), torch.bfloat16),                    # 2 MiB on the wire: eager, several CTAs
            (torch.randn(3 << 20, device="cuda:0"), torch.bfloat16),                    # 6 MiB on the wire: eager, a run of six slots
            (torch.randn(1 << 24, device="cuda:0"), torch.bfloat16),                    # 32 MiB on the wire: converted by the receiver's pull
            (torch.randn(1 << 24, device="cuda:0")[3:], torch.float16),                 # an unaligned start: the element-wise kernel
            (torch.randn(2048, 1500, device="cuda:0").t(), torch.bfloat16),             # strided and converted at once
            (torch.randn(4096, device="cuda:0").to(torch.bfloat16), torch.float32),     # widening
        ]
        for x, wire in cases:
            y = await client.invoke(x, worker_name="cv_server", session_id=1, function="what_arrived", memory_policy=on_device, wire_dtype=wire)
            assert seen[-1] == (wire, tuple(x.shape)), (seen[-1], wire, x.shape)
            assert y.dtype == wire and y.shape == x.shape
            assert torch.equal(y, x.contiguous().to(wire)), (x.shape, x.dtype, wire)
            del y
        st = client.transport_stats()
        assert st["device_packs"] == 0 and st["device_staged"] == 0, st
        # the same value without wire_dtype travels as it is
        x = torch.randn(1000, device="cuda:0")
        y = await client.invoke(x, worker_name="cv_server", session_id=1, function="what_arrived", memory_policy=on_device)
        assert y.dtype == torch.float32 and torch.equal(y, x)
        # a function whose fp32 results travel as bf16
        x = torch.randn(1 << 22, device="cuda:0").to(torch.bfloat16)
        y = await client.invoke(x, worker_name="cv_server", session_id=1, function="as_fp32", memory_policy=on_device)
        assert y.dtype == torch.bfloat16 and torch.equal(y, (x.float() * 2.0).to(torch.bfloat16))
        # host tensors are converted before they are sent
        h = torch.randn(64)
        y = await client.invoke(h, worker_name="cv_server", session_id=1, function="what_arrived", wire_dtype=torch.bfloat16)
        assert y.dtype == torch.bfloat16 and torch.equal(y.cpu(), h.to(torch.bfloat16))
        client.stop()
        server.stop()

    run(main())


def test_many_mixed_calls_in_flight(cuda_device):
    """Several hundred calls of random size (256 B to 24 MiB), dense, strided or converted, up to 24 in flight at
    once, between a client and a server runtime: eager runs of ring slots, pulls, pushes and held announcements
    all mix, slots run out and come back, and every reply is checked."""
    import random

    from execution_ucx_b200 import axon

    async def main():
        server = axon.AxonRuntime("mix_server", timeout=60000, device=axon.cuda(0))
        client = axon.AxonRuntime("mix_client", timeout=60000, device=axon.cuda(0))
        table = {(2, 32): torch.float32, (2, 16): torch.float16, (4, 16): torch.bfloat16}

        def on_device(metas):
            m = metas[0]
            return torch.empty(m.shape, dtype=table[(m.dtype.code, m.dtype.bits)], device="cuda:0")

        async def scale(x: torch.Tensor, k: float) -> torch.Tensor:
            return x * k

        server.register_function(scale, memory_policy=on_device)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "mix_server")
        rng = random.Random(1234)
        sem = asyncio.Semaphore(24)
        failures = []

        async def one(i: int):
            async with sem:
                kind = rng.choice(("dense", "dense", "strided", "cast", "fresh"))
                n = int(2 ** rng.uniform(6, 22.5))                       # elements
                if kind == "strided":
                    rows = max(2, int(n ** 0.5))
                    x = torch.randn(rows, rows + 3, device="cuda:0")[:, 1:-2].t()
                    want_dtype, wire = torch.float32, None
                elif kind == "cast":
                    x = torch.randn(n, device="cuda:0")
                    want_dtype, wire = torch.bfloat16, torch.bfloat16
                elif kind == "fresh":
                    # produced on a side stream right before the call: the send must wait for it on the device
                    s = torch.cuda.Stream(device="cuda:0")
                    s.wait_stream(torch.cuda.current_stream())
                    with torch.cuda.stream(s):
                        x = torch.zeros(n, device="cuda:0")
                        torch.cuda._sleep(2_000_000)
                        x.add_(float(i % 97))
                        fut = client.invoke(x, 2.0, worker_name="mix_server", session_id=i, function="scale", memory_policy=on_device)
                    y = await fut
                    torch.cuda.current_stream().wait_stream(s)
                    if not (float(y.min()) == float(y.max()) == 2.0 * (i % 97)):
                        failures.append((i, kind, n, float(y.min()), float(y.max())))
                    return
                else:
                    x = torch.randn(n, device="cuda:0")
                    want_dtype, wire = torch.float32, None
                y = await client.invoke(x, 2.0, worker_name="mix_server", session_id=i, function="scale", memory_policy=on_device, wire_dtype=wire)
                ref = (x.contiguous().to(want_dtype) * 2.0)
                if y.dtype != want_dtype or y.shape != x.shape or not torch.equal(y, ref):
                    failures.append((i, kind, tuple(x.shape), y.dtype))

        await asyncio.gather(*[one(i) for i in range(400)])
        assert not failures, failures[:5]
        cs, ss = client.transport_stats(), server.transport_stats()
        assert cs["device_staged"] == 0 and ss["device_staged"] == 0, (cs, ss)
        assert cs["device_eager_sent"] > 0 and cs["device_pushes"] + ss["device_pulls"] > 0, (cs, ss)
        client.stop()
        server.stop()

    run(main())


def test_many_mixed_calls_between_processes():
    """The same mix against a server in another process (on GPU 1 where there is one): the payloads cross
    through mapped peer memory, the flags through the shared page, and slots come back through the segment."""
    import random

    server_dev = 1 if torch.cuda.device_count() > 1 else 0
    env = dict(os.environ, PYTHONPATH=str(ROOT), NCCL_NVLS_ENABLE="0")
    child = subprocess.Popen([sys.executable, "-m", "execution_ucx_b200.models.echo_server", "--device", str(server_dev), "--name", "mix_peer",
                              "--timeout-ms", "60000"], stdout=subprocess.PIPE, stdin=subprocess.PIPE, env=env, cwd=str(ROOT))
    try:
        line = child.stdout.readline().decode().strip()
        assert line.startswith("ADDRESS "), line
        address = bytes.fromhex(line.split()[1])
        from execution_ucx_b200 import axon

        async def main():
            client = axon.AxonRuntime("mix_client2", timeout=60000, device=axon.cuda(0))
            client.start_client()
            await client.connect_endpoint_async(address, "mix_peer")
            table = {(2, 32): torch.float32, (2, 16): torch.float16, (4, 16): torch.bfloat16}

            def on_device(metas):
                m = metas[0]
                return torch.empty(m.shape, dtype=table[(m.dtype.code, m.dtype.bits)], device="cuda:0")

            rng = random.Random(99)
            sem = asyncio.Semaphore(24)
            failures = []

            async def one(i: int):
                async with sem:
                    kind = rng.choice(("dense", "dense", "strided", "cast"))
                    n = int(2 ** rng.uniform(6, 22.5))
                    wire = None
                    if kind == "strided":
                        rows = max(2, int(n ** 0.5))
                        x = torch.randn(rows, rows + 3, device="cuda:0")[:, 1:-2].t()
                    else:
                        x = torch.randn(n, device="cuda:0")
                        if kind == "cast":
                            wire = torch.bfloat16
                    y = await client.invoke(x, worker_name="mix_peer", session_id=i, function="add_one", memory_policy=on_device, wire_dtype=wire)
                    ref = x.contiguous().to(wire or torch.float32) + 1.0
                    if y.dtype != ref.dtype or y.shape != x.shape or not torch.equal(y, ref):
                        failures.append((i, kind, tuple(x.shape), y.dtype))

            await asyncio.gather(*[one(i) for i in range(300)])
            assert not failures, failures[:5]
            st = client.transport_stats()
            assert st["device_staged"] == 0 and st["device_eager_sent"] > 0 and st["device_packs"] == 0, st
            client.stop()

        run(main())
    finally:
        try:
            child.stdin.write(b"quit\n")
            child.stdin.flush()
            child.wait(timeout=30)
        except Exception:
            child.kill()
