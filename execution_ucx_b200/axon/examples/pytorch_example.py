"""Two runtimes in one process exchanging CPU tensors (the counterpart of the reference's
axon/python/examples/pytorch_example.py).

    python -m execution_ucx_b200.axon.examples.pytorch_example

A server registers three functions from their annotations; a client calls them with scalars,
one tensor, and a list of tensors. Small payloads travel inside the message (eager), large ones
are announced first and then fetched into the buffer that the memory policy hands out.
"""
from __future__ import annotations

import asyncio
from typing import List, Tuple

import torch

from execution_ucx_b200 import axon


async def main() -> None:
    server = axon.AxonRuntime("example_server", timeout=5000)
    client = axon.AxonRuntime("example_client", timeout=5000)

    async def scale_add(x: torch.Tensor, scale: float, bias: int) -> torch.Tensor:
        return x * scale + bias

    async def stats(x: torch.Tensor) -> Tuple[float, float, int]:
        return float(x.mean()), float(x.std()), x.numel()

    async def add_all(xs: List[torch.Tensor], names: List[str]) -> List[torch.Tensor]:
        print("  server got", names)
        return [x + 1 for x in xs]

    for fn in (scale_add, stats, add_all):
        server.register_function(fn)
    server.start_server()
    client.start_client()
    await client.connect_endpoint_async(server.get_local_address(), "example_server")
    # what the server offers, as the client can learn it
    for sig in axon.deserialize_signatures(server.get_local_signatures()):
        print("  offers", sig.function_name, sig.id)

    x = torch.arange(8, dtype=torch.float32)
    y = await client.invoke(x, 2.0, 1, worker_name="example_server", session_id=1, function="scale_add")
    print("scale_add (eager):", y.tolist())

    received_in = []

    def policy(metas):
        t = torch.empty(metas[0].shape, dtype=torch.float32)
        received_in.append(t)
        return t

    big = torch.rand(1 << 20)
    y = await client.invoke(big, 0.5, 0, worker_name="example_server", session_id=1, function="scale_add", memory_policy=policy)
    print("scale_add (rendezvous): result is the tensor the policy returned:", y is received_in[-1],
          "max err", float((y - big * 0.5).abs().max()))

    mean, std, n = await client.invoke(big, worker_name="example_server", session_id=1, function="stats")
    print(f"stats: mean={mean:.4f} std={std:.4f} n={n}")

    outs = await client.invoke([torch.zeros(3), torch.ones(5)], ["zeros", "ones"], worker_name="example_server",
                               session_id=1, function="add_all")
    print("add_all:", [o.tolist() for o in outs])
    client.stop()
    server.stop()


if __name__ == "__main__":
    asyncio.run(main())
