"""A stand-alone Axon echo server: prints ``ADDRESS <hex>`` on stdout, serves ``echo`` and
``add_one`` for device tensors until ``quit`` arrives on stdin; ``stats`` on stdin is answered with
``STATS <json of the transport counters>``.

    python -m execution_ucx_b200.models.echo_server --device 1 --name peer
"""
from __future__ import annotations

import argparse
import asyncio
import sys

import torch


async def _serve(args) -> None:
    from .. import axon
    dev = f"cuda:{args.device}"
    torch.cuda.set_device(args.device)
    rt = axon.AxonRuntime(args.name, timeout=args.timeout_ms, device=axon.cuda(args.device))
    dtype_by_bits = {(4, 16): torch.bfloat16, (2, 16): torch.float16, (2, 32): torch.float32, (1, 8): torch.uint8}

    def on_device(metas):
        outs = [torch.empty(m.shape, dtype=dtype_by_bits[(m.dtype.code, m.dtype.bits)], device=dev) for m in metas]
        return outs if len(outs) > 1 else outs[0]

    async def echo(x: torch.Tensor) -> torch.Tensor:
        return x

    async def add_one(x: torch.Tensor) -> torch.Tensor:
        return x + 1.0

    rt.register_function(echo, memory_policy=on_device)
    rt.register_function(add_one, memory_policy=on_device)
    rt.start_server()
    print("ADDRESS " + rt.get_local_address().hex(), flush=True)
    loop = asyncio.get_running_loop()
    while True:
        line = await loop.run_in_executor(None, sys.stdin.readline)
        if not line or line.strip() == "quit":
            break
        if line.strip() == "stats":
            import json
            print("STATS " + json.dumps(rt.transport_stats()), flush=True)
    rt.stop()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--device", type=int, default=0)
    ap.add_argument("--name", default="echo_server")
    ap.add_argument("--timeout-ms", type=int, default=20000)
    asyncio.run(_serve(ap.parse_args()))


if __name__ == "__main__":
    main()
