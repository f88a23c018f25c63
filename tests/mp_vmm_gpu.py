"""Client half of the expandable-segments test (run as a script in a process of its own, because the
allocator's configuration is read once, at the first CUDA allocation): tensors whose memory the tensor
library made with cuMemCreate and mapped 20 MiB at a time have no CUDA IPC handle; they must still cross
between processes on the device paths, by file descriptors handed over a Unix socket."""
import asyncio
import json
import os
import subprocess
import sys
from pathlib import Path

import torch

ROOT = Path(__file__).resolve().parent.parent


def main() -> int:
    assert "expandable_segments:True" in os.environ.get("PYTORCH_CUDA_ALLOC_CONF", "")
    server_dev = 1 if torch.cuda.device_count() > 1 else 0
    child = subprocess.Popen([sys.executable, "-m", "execution_ucx_b200.models.echo_server", "--device", str(server_dev), "--name", "vmm_peer"],
                             stdout=subprocess.PIPE, stdin=subprocess.PIPE, env=dict(os.environ, PYTHONPATH=str(ROOT)), cwd=str(ROOT))
    try:
        line = child.stdout.readline().decode().strip()
        assert line.startswith("ADDRESS "), line
        address = bytes.fromhex(line.split()[1])
        from execution_ucx_b200 import axon

        async def run():
            client = axon.AxonRuntime("vmm_client", timeout=20000, device=axon.cuda(0))
            client.start_client()
            await client.connect_endpoint_async(address, "vmm_peer")
            policy = lambda metas: torch.empty(metas[0].shape, dtype=torch.bfloat16, device="cuda:0")  # noqa: E731
            # (the eager limit is 64 KiB in this test) 2 KiB: eager into the peer's ring; 2 MiB: pulled out of this process's segments by the peer's
            # kernel; 96 MiB: pushed into the peer's segments (five 20 MiB allocations under one tensor), and
            # back the same ways
            for n in (1024, 1 << 20, 48 << 20):
                x = torch.randn(n, device="cuda:0").to(torch.bfloat16)
                y = await client.invoke(x, worker_name="vmm_peer", session_id=1, function="echo", memory_policy=policy)
                assert y.device.index == 0 and torch.equal(y.view(torch.int16), x.view(torch.int16)), n
                del y
            # a 3 MiB window (pulled, not pushed) that starts in one allocation and ends in the next, at an odd offset
            from cuda.bindings import driver as cu
            big = torch.randn(30 << 20, device="cuda:0").to(torch.bfloat16)
            err, base, size = cu.cuMemGetAddressRange(big.data_ptr())
            assert err == cu.CUresult.CUDA_SUCCESS
            boundary = (int(base) + int(size) - big.data_ptr()) // 2      # first element of the next allocation
            assert 0 < boundary < big.numel() - (1 << 20), (boundary, big.numel())
            start = max(0, boundary - (1 << 19) - 5)
            part = big[start:start + (3 << 19)]
            assert part.data_ptr() < int(base) + int(size) < part.data_ptr() + part.numel() * 2
            y = await client.invoke(part, worker_name="vmm_peer", session_id=1, function="echo", memory_policy=policy)
            assert torch.equal(y.view(torch.int16), part.view(torch.int16))
            st = client.transport_stats()
            client.stop()
            return st

        loop = asyncio.new_event_loop()
        asyncio.set_event_loop(loop)
        st = loop.run_until_complete(run())
        child.stdin.write(b"stats\n")
        child.stdin.flush()
        line = child.stdout.readline().decode().strip()
        assert line.startswith("STATS "), line
        peer = json.loads(line[6:])
        print("client", json.dumps(st))
        print("server", json.dumps(peer))
        for who, s in (("client", st), ("server", peer)):
            assert s["device_staged"] == 0, (who, s)
            assert s["vmm_fds_sent"] > 0 and s["vmm_fds_recv"] > 0, (who, s)
        assert st["device_eager_sent"] == 1 and st["device_pushes"] == 1 and st["device_push_recv"] == 1, st
        assert peer["device_pulls"] == 2 and st["device_pulls"] == 2, (st, peer)   # 2 MiB and the 3 MiB window, there and back
        # the 96 MiB tensor lies in at least five allocations, each handed over once
        assert st["vmm_fds_recv"] >= 5 and peer["vmm_fds_recv"] >= 1, (st, peer)
        print("OK")
        return 0
    finally:
        try:
            child.stdin.write(b"quit\n")
            child.stdin.flush()
            child.wait(timeout=30)
        except Exception:
            child.kill()


if __name__ == "__main__":
    sys.exit(main())
