"""The RPC workload of the benchmark on two gloo ranks with host tensors: each rank serves `echo`
and calls it on its partner through AxonRuntime.invoke (host-side logic only, no GPU)."""
import os
import subprocess
import sys
from pathlib import Path

ROOT = Path(__file__).resolve().parent.parent

CHILD = r"""
import asyncio, os, sys
import torch, torch.distributed as dist
from execution_ucx_b200.models.workloads import AxonTensorRpc
from execution_ucx_b200.parallel.peer import PeerGroup

dist.init_process_group("gloo")
group = PeerGroup(dist.get_rank(), dist.get_world_size(), torch.device("cpu"))

async def main():
    w = AxonTensorRpc(group, dtype=torch.float32, timeout_ms=20000)
    await w.start()
    for n in (16, 5000, 1 << 18):
        x = torch.rand(n) + group.rank
        for _ in range(3):
            y = await w.step(x)
            assert torch.equal(y, x), (group.rank, n)
        await w.barrier()
    w.stop()

asyncio.run(main())
dist.barrier()
dist.destroy_process_group()
print("RANK_OK", flush=True)
"""


def test_axon_workload_two_gloo_ranks(tmp_path):
    script = tmp_path / "child.py"
    script.write_text(CHILD)
    env = dict(os.environ, PYTHONPATH=str(ROOT), MASTER_ADDR="127.0.0.1")
    out = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2",
                          "--master-addr", "127.0.0.1", "--master-port", "29541", str(script)],
                         env=env, cwd=str(ROOT), capture_output=True, text=True, timeout=240)
    assert out.returncode == 0, out.stdout[-3000:] + out.stderr[-3000:]
    assert out.stdout.count("RANK_OK") == 2
