"""CUDA tensors through the RPC runtime (the counterpart of the reference's
axon/python/examples/pytorch_cuda_example.py).

    python -m execution_ucx_b200.axon.examples.pytorch_cuda_example [--peer-device 1]

With ``--peer-device N`` the server runs in a child process on GPU N and the tensors cross NVLink;
without it both runtimes share GPU 0. Device payloads never pass through host memory: the receiver
maps the sender's allocation and copies with the transfer kernel, straight into the tensor that
the memory policy returned (so the result *is* that tensor).
"""
from __future__ import annotations

import argparse
import asyncio
import subprocess
import sys

import torch

from execution_ucx_b200 import axon


async def run(peer_device: int | None) -> None:
    if not torch.cuda.is_available():
        print("no CUDA device: this example needs a GPU")
        return
    torch.cuda.set_device(0)
    child = None
    client = axon.AxonRuntime("cuda_client", timeout=20000, device=axon.cuda(0))
    if peer_device is None:
        server = axon.AxonRuntime("cuda_server", timeout=20000, device=axon.cuda(0))

        async def add_one(x: torch.Tensor) -> torch.Tensor:
            return x + 1.0

        server.register_function(add_one, memory_policy=lambda metas: torch.empty(metas[0].shape, dtype=torch.float32, device="cuda:0"))
        server.start_server()
        address, name = server.get_local_address(), "cuda_server"
    else:
        child = subprocess.Popen([sys.executable, "-m", "execution_ucx_b200.models.echo_server", "--device", str(peer_device),
                                  "--name", "cuda_server"], stdout=subprocess.PIPE, stdin=subprocess.PIPE)
        line = child.stdout.readline().decode().split()
        address, name = bytes.fromhex(line[1]), "cuda_server"
    client.start_client()
    await client.connect_endpoint_async(address, name)

    handed_out = []

    def policy(metas):
        t = torch.empty(metas[0].shape, dtype=torch.float32, device="cuda:0")
        handed_out.append(t)
        return t

    for n in (1024, 1 << 24):
        x = torch.rand(n, device="cuda:0")
        y = await client.invoke(x, worker_name=name, session_id=1, function="add_one", memory_policy=policy)
        # a small result arrives eagerly in the runtime's receive ring (the policy is not asked); a large one
        # lands in the tensor that the policy handed out, and that very object is the result
        where = "the policy's tensor" if handed_out and y is handed_out[-1] else "the receive ring"
        print(f"add_one({n} floats): on {y.device}, received into {where}, max err {float((y - (x + 1)).abs().max()):.1e}")
    client.stop()
    if child is None:
        server.stop()
    else:
        child.stdin.write(b"quit\n")
        child.stdin.flush()
        child.wait(timeout=30)


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--peer-device", type=int, default=None)
    asyncio.run(run(ap.parse_args().peer_device))
