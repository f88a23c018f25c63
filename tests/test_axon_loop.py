"""The spinning event loop: calls complete on it, timers and other file descriptors keep working."""
import asyncio
import socket
import time

import numpy as np
import pytest


@pytest.fixture(scope="module")
def axon(native_build):
    from execution_ucx_b200 import axon as ax
    return ax


def test_spin_returns_when_nothing_is_queued(axon):
    t0 = time.perf_counter()
    assert axon._axon._spin_for_wake(0.002) is False
    spent = time.perf_counter() - t0
    assert 0.0015 <= spent < 0.5
    assert axon._axon._spin_for_wake(0.0) is False
    with pytest.raises(ValueError):
        axon.SpinningSelector(-1)


def test_calls_timers_and_sockets_on_the_spinning_loop(axon):
    async def main():
        server = axon.AxonRuntime("loop_srv", timeout=5000)
        client = axon.AxonRuntime("loop_cli", timeout=5000)

        async def twice(x: np.ndarray, k: int) -> np.ndarray:
            await asyncio.sleep(0)          # the handler goes through the loop once itself
            return x * k

        server.register_function(twice, from_dlpack_fn=np.from_dlpack)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "loop_srv")
        x = np.arange(1024, dtype=np.float32)
        for k in range(1, 40):
            y = await client.invoke(x, k, worker_name="loop_srv", session_id=k, function="twice", from_dlpack_fn=np.from_dlpack)
            assert np.array_equal(y, x * k)
        many = await asyncio.gather(*[client.invoke(x, 3, worker_name="loop_srv", session_id=100 + i, function="twice",
                                                    from_dlpack_fn=np.from_dlpack) for i in range(32)])
        assert all(np.array_equal(y, x * 3) for y in many)

        # a timer shorter and one longer than the spin
        for delay in (0.00005, 0.02):
            t0 = time.perf_counter()
            await asyncio.sleep(delay)
            assert delay <= time.perf_counter() - t0 < delay + 0.25

        # a descriptor that has nothing to do with the runtime is still served
        a, b = socket.socketpair()
        a.setblocking(False)
        b.setblocking(False)
        loop = asyncio.get_running_loop()
        got = loop.create_future()
        loop.add_reader(a.fileno(), lambda: got.set_result(a.recv(16)))
        loop.call_later(0.005, b.send, b"ping")
        assert await asyncio.wait_for(got, 5) == b"ping"
        loop.remove_reader(a.fileno())
        a.close()
        b.close()
        client.stop()
        server.stop()
        return type(loop._selector).__name__

    assert axon.run(main(), spin_us=200) == "SpinningSelector"
    # the same through asyncio.run and with the spin switched off
    assert asyncio.run(main(), loop_factory=lambda: axon.new_event_loop(0)) == "SpinningSelector"
