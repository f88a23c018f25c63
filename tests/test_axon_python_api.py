"""More of the Python API: timeouts in all accepted forms, deadlines, error text, nested lists and
string lists, signatures discovery, awaited handlers, concurrency, stop/start and unknown workers."""
import asyncio
import datetime
from typing import List, Tuple

import numpy as np
import pytest


@pytest.fixture(scope="module")
def axon(native_build):
    from execution_ucx_b200 import axon as ax
    return ax


def run(coro):
    loop = asyncio.new_event_loop()
    try:
        asyncio.set_event_loop(loop)
        return loop.run_until_complete(coro)
    finally:
        loop.close()


def test_timeout_forms_and_strict_registration(axon):
    for t in (250, 0.25, datetime.timedelta(milliseconds=250), None):
        rt = axon.AxonRuntime("t_forms", timeout=t)
        rt.stop()
    with pytest.raises(TypeError):
        axon.AxonRuntime("bad_timeout", timeout="soon")
    rt = axon.AxonRuntime("strict", timeout=1000)

    def not_async(x: int) -> int:
        return x

    async def no_annotation(x) -> int:
        return 1

    with pytest.raises(RuntimeError, match="only accepts async functions"):   # the reference's exception type and text
        rt.register_function(not_async)
    with pytest.raises(TypeError, match="Unsupported or missing type annotation for parameter 0"):
        rt.register_function(no_annotation)
    rt.register_function_raw(function_id=900, callable=no_annotation)       # the raw form tolerates it (UNKNOWN)

    async def ok(x: int) -> int:
        return x

    fid = rt.register_function(ok)
    assert fid == axon.function_id_from_name("ok", "strict")
    with pytest.raises(ValueError):
        rt.register_function(ok)       # the id is taken
    rt.stop()


def test_values_lists_errors_and_deadline(axon):
    async def main():
        server = axon.AxonRuntime("api_server", timeout=3000)
        client = axon.AxonRuntime("api_client", timeout=300)
        seen = {}

        async def mix(flag: bool, n: int, x: float, s: str, ints: List[int], floats: List[float], names: List[str]) -> Tuple[bool, int, float, str, List[int], List[str]]:
            seen["args"] = (flag, n, x, s, ints, floats, names)
            return (not flag, n + 1, x * 2, s.upper(), [i * 2 for i in ints], list(reversed(names)))

        async def nested(groups: List[List[int]]) -> int:
            return sum(sum(g) for g in groups)

        async def slow(ms: int) -> int:
            await asyncio.sleep(ms / 1000.0)
            return ms

        async def fails(n: int) -> int:
            raise KeyError("missing %d" % n)

        for fn in (mix, nested, slow, fails):
            server.register_function(fn)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "api_server")
        call = lambda fn, *a: client.invoke(*a, worker_name="api_server", session_id=7, function=fn)  # noqa: E731

        out = await call("mix", True, 41, 1.5, "abc", [1, 2, 3], [0.5, 0.25], ["x", "yy", ""])
        assert out == (False, 42, 3.0, "ABC", [2, 4, 6], ["", "yy", "x"])
        assert seen["args"] == (True, 41, 1.5, "abc", [1, 2, 3], [0.5, 0.25], ["x", "yy", ""])
        assert await call("nested", [[1, 2], [], [3, 4, 5]]) == 15

        # an awaited handler below the deadline, then one above it
        assert await call("slow", 50) == 50
        with pytest.raises(RuntimeError) as err:
            await call("slow", 800)
        assert "deadline" in str(err.value).lower()

        # the remote exception's text comes back with the ids of the call
        with pytest.raises(RuntimeError) as err:
            await call("fails", 9)
        text = str(err.value)
        assert "missing 9" in text and "(session_id: 7)" in text
        assert "(function_id: %d)" % axon.function_id_from_name("fails", "api_server") in text

        # unknown function, unknown worker
        with pytest.raises(RuntimeError):
            await call("no_such_function", 1)
        with pytest.raises(Exception):
            await client.invoke(1, worker_name="nobody", session_id=1, function="mix")

        # many calls in flight
        results = await asyncio.gather(*[call("nested", [[i], [i, i]]) for i in range(200)])
        assert results == [3 * i for i in range(200)]

        # what the server offers, from its signature blob
        sigs = {s.function_name: s for s in axon.deserialize_signatures(server.get_local_signatures())}
        assert set(sigs) == {"mix", "nested", "slow", "fails"}
        assert sigs["slow"].id == axon.function_id_from_name("slow", "api_server")
        client.stop()
        server.stop()

    run(main())


def test_tensor_lists_and_mixed_returns(axon):
    async def main():
        server = axon.AxonRuntime("tl_server", timeout=5000)
        client = axon.AxonRuntime("tl_client", timeout=5000)

        async def split(x: np.ndarray, parts: int) -> List[np.ndarray]:
            return [np.ascontiguousarray(p) for p in np.array_split(x, parts)]

        async def describe(xs: List[np.ndarray]) -> Tuple[int, np.ndarray]:
            return len(xs), np.concatenate([a.ravel() for a in xs]).astype(np.float32)

        server.register_function(split)
        server.register_function(describe)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "tl_server")
        x = np.arange(100000, dtype=np.float32)
        parts = await client.invoke(x, 3, worker_name="tl_server", session_id=1, function="split")
        assert len(parts) == 3 and np.array_equal(np.concatenate(parts), x)
        n, flat = await client.invoke([np.ones((2, 3), dtype=np.float32), np.zeros(5, dtype=np.float32)], worker_name="tl_server",
                                      session_id=1, function="describe")
        assert n == 2 and flat.tolist() == [1.0] * 6 + [0.0] * 5
        # stop and start again: the same runtimes serve a new connection
        client.stop_client()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "tl_server")
        parts = await client.invoke(x[:10], 2, worker_name="tl_server", session_id=1, function="split")
        assert [p.tolist() for p in parts] == [x[:5].tolist(), x[5:10].tolist()]
        client.stop()
        server.stop()

    run(main())
