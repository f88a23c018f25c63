"""Child process of test_axon_python_lifetime.py: runtimes are stopped, dropped and cancelled with calls in
flight, from the event loop's own thread (where a stop() that waited for the loop would wait for ever)."""
import asyncio
import gc
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))
import numpy as np  # noqa: E402

from execution_ucx_b200 import axon  # noqa: E402

small = np.arange(1 << 12, dtype=np.float32)
big = np.arange(1 << 18, dtype=np.float32)      # 1 MiB: a rendezvous that is still arriving when the stop comes


async def pair(tag: str):
    server = axon.AxonRuntime("s" + tag, timeout=2000)
    client = axon.AxonRuntime("c" + tag, timeout=2000)

    async def slow(x: np.ndarray, delay: float) -> np.ndarray:
        await asyncio.sleep(delay)
        return x + 1

    server.register_function(slow, from_dlpack_fn=np.from_dlpack)
    server.start_server()
    client.start_client()
    await client.connect_endpoint_async(server.get_local_address(), "s" + tag)
    return server, client


def call(client, tag, x, delay):
    return client.invoke(x, delay, worker_name="s" + tag, session_id=1, function="slow", from_dlpack_fn=np.from_dlpack)


async def settle(futures, limit):
    for f in futures:
        try:
            await asyncio.wait_for(f, limit)
        except Exception:
            pass


async def scenario(i: int):
    tag = str(i)
    server, client = await pair(tag)
    kind = i % 5
    try:
        if kind == 0:      # the client stops with calls in flight; the server stops while their payloads still arrive
            futures = [call(client, tag, big, 0.2) for _ in range(8)]
            client.stop()
            await settle(futures, 1)
        elif kind == 1:    # the server stops while its handlers sleep
            futures = [call(client, tag, small, 0.3) for _ in range(8)]
            await asyncio.sleep(0.05)
            server.stop()
            await settle(futures, 3)
        elif kind == 2:    # the callers are cancelled; the pair still works afterwards
            tasks = [asyncio.ensure_future(call(client, tag, big, 0.2)) for _ in range(8)]
            await asyncio.sleep(0.01)
            for t in tasks:
                t.cancel()
            await asyncio.gather(*tasks, return_exceptions=True)
            assert np.array_equal(await call(client, tag, small, 0.0), small + 1)
        elif kind == 3:    # both runtimes are dropped without a stop, calls in flight
            futures = [call(client, tag, big, 0.1) for _ in range(4)]
            del server, client
            gc.collect()
            await settle(futures, 1)
            return
        else:              # only the server half stops, with requests queued for the loop
            futures = [call(client, tag, big, 0.2) for _ in range(8)]
            server.stop_server()
            await settle(futures, 3)
    finally:
        try:
            client.stop()
            server.stop()
        except NameError:
            pass


async def main(rounds: int):
    for i in range(rounds):
        await asyncio.wait_for(scenario(i), 30)


if __name__ == "__main__":
    asyncio.run(main(int(sys.argv[1])))
    print("OK")
