"""Lifetimes and layouts on the Python API: who keeps a tensor's bytes alive and for how long, what
happens to views and strided inputs, and which element types travel (CPU only, numpy tensors).

The reference covers the same ground in axon/python/tests/test_numpy_rpc.py:471-572 (lifetime) and
test_invoke_memory_policy.py:50-104."""
import asyncio
import gc
import weakref

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


async def _pair(axon, name, register):
    server = axon.AxonRuntime(name + "_server", timeout=5000)
    client = axon.AxonRuntime(name + "_client", timeout=5000)
    register(server)
    server.start_server()
    client.start_client()
    await client.connect_endpoint_async(server.get_local_address(), name + "_server")
    return server, client


def test_results_outlive_the_runtimes(axon):
    """A result tensor (small: inline, large: rendezvous) stays readable after both runtimes were stopped
    and dropped: the buffer under it keeps its memory resource alive."""
    async def main():
        async def ramp(n: int, start: float) -> np.ndarray:
            return np.arange(n, dtype=np.float32) + np.float32(start)

        server, client = await _pair(axon, "life", lambda s: s.register_function(ramp))
        call = lambda n, s: client.invoke(n, s, worker_name="life_server", session_id=1, function="ramp")  # noqa: E731
        small = await call(16, 1.0)
        large = await call(300_000, 2.0)
        client.stop()
        server.stop()
        return small, large

    small, large = run(main())
    gc.collect()
    np.testing.assert_array_equal(small, np.arange(16, dtype=np.float32) + 1)
    np.testing.assert_array_equal(large, np.arange(300_000, dtype=np.float32) + 2)
    # and they can be copied and computed on like any other array
    more = large.copy()
    more += 1
    assert float(more[-1]) == 300_000 + 2 and float(large[-1]) == 300_000 + 1


def test_request_tensor_may_be_dropped_by_the_caller(axon):
    """The caller deletes its only reference to the request tensor right after `invoke`: the call still
    delivers the bytes, and the tensor is released once the call is over."""
    async def main():
        async def total(x: np.ndarray) -> float:
            return float(x.sum(dtype=np.float64))

        server, client = await _pair(axon, "drop", lambda s: s.register_function(total))
        dead = []
        futures = []
        for n in (64, 400_000):
            x = np.full(n, 0.5, dtype=np.float32)
            dead.append(weakref.ref(x))
            futures.append(client.invoke(x, worker_name="drop_server", session_id=1, function="total"))
            del x
        gc.collect()
        results = [await f for f in futures]
        assert results == [32.0, 200_000.0]
        # nothing keeps the request tensors once their calls have completed (a few loop turns for the
        # transport to let go of the send buffers)
        for _ in range(50):
            gc.collect()
            if all(r() is None for r in dead):
                break
            await asyncio.sleep(0.01)
        assert all(r() is None for r in dead)
        client.stop()
        server.stop()

    run(main())


def test_views_strides_and_forwarding(axon):
    """Strided and transposed inputs arrive dense with the right values; a read-only view of a received
    tensor can be returned by the handler (it travels as a copy); a handler may return its own input."""
    async def main():
        seen = {}

        async def head(x: np.ndarray, n: int) -> np.ndarray:
            seen["contiguous"] = bool(x.flags["C_CONTIGUOUS"])
            v = x[:n]
            v.flags.writeable = False
            return v

        async def same(x: np.ndarray) -> np.ndarray:
            return x

        def reg(s):
            s.register_function(head)
            s.register_function(same)

        server, client = await _pair(axon, "view", reg)
        base = np.arange(2 * 50_000, dtype=np.float32).reshape(50_000, 2)
        every_other = base[:, 0]                      # stride of two elements
        out = await client.invoke(every_other, 10, worker_name="view_server", session_id=1, function="head")
        np.testing.assert_array_equal(out, every_other[:10])
        assert seen["contiguous"]
        mat = np.arange(12, dtype=np.int32).reshape(3, 4)
        back = await client.invoke(mat.T, worker_name="view_server", session_id=1, function="same")
        assert back.shape == (4, 3)
        np.testing.assert_array_equal(back, mat.T)
        big = np.arange(150_000, dtype=np.float64)
        back = await client.invoke(big, worker_name="view_server", session_id=1, function="same")
        np.testing.assert_array_equal(back, big)
        assert back is not big
        client.stop()
        server.stop()

    run(main())


@pytest.mark.parametrize("dtype", ["uint8", "int8", "int16", "int32", "int64", "float16", "float32", "float64", "bool"])
def test_element_types_round_trip(axon, dtype):
    """Every numpy element type that DLPack can describe comes back bit for bit, inline and by rendezvous,
    and its metadata names the same type."""
    async def main():
        async def echo(x: np.ndarray) -> np.ndarray:
            return x

        server, client = await _pair(axon, "dt_" + dtype, lambda s: s.register_function(echo))
        rng = np.random.default_rng(3)
        for n in (33, 70_000):
            if dtype == "bool":
                x = rng.integers(0, 2, n).astype(np.bool_)
            elif dtype.startswith("float"):
                x = rng.standard_normal(n).astype(dtype)
            else:
                info = np.iinfo(dtype)
                x = rng.integers(info.min, info.max, n, dtype=dtype, endpoint=True)
            m = axon.TensorMeta.from_tensor(x)
            assert m.shape == [n] and m.nbytes() == x.nbytes
            y = await client.invoke(x, worker_name="dt_" + dtype + "_server", session_id=1, function="echo")
            assert y.dtype == x.dtype and y.shape == x.shape
            assert y.tobytes() == x.tobytes()
        client.stop()
        server.stop()

    run(main())


def test_devices_and_context_handle(axon):
    """The device descriptors and the context-handle query work on a machine without a GPU."""
    assert axon.cpu().kind == "cpu" and str(axon.cpu()) in ("cpu", "cpu:0")
    d = axon.cuda(3)
    assert isinstance(d, axon.CudaDevice) and d.kind == "cuda" and d.index == 3
    assert axon.rocm(1).kind == "rocm" and axon.sycl(0).kind == "sycl"
    assert isinstance(axon.auto_detect(), axon.Device)
    h = axon.get_device_context_handle("cuda")
    assert h is None or isinstance(h, int)
    with pytest.raises(ValueError):
        axon.AxonRuntime("bad_device", device=axon.rocm(0))


def test_stop_drop_and_cancel_with_calls_in_flight(native_build):
    """stop() runs on the event loop's thread and waits for every call to be answered: requests that were queued
    for the loop at that moment used to wait for the loop in turn. Forty rounds of stopping, dropping and
    cancelling with calls in flight, in a process of its own so that a deadlock shows as a timeout."""
    import os
    import subprocess
    import sys
    from pathlib import Path

    root = Path(__file__).resolve().parent.parent
    env = dict(os.environ, PYTHONPATH=str(root), EUX_LOG_LEVEL="OFF")
    out = subprocess.run([sys.executable, str(root / "tests" / "mp_stop_in_flight.py"), "40"], env=env, cwd=str(root),
                         capture_output=True, text=True, timeout=240)
    assert out.returncode == 0 and out.stdout.strip().endswith("OK"), out.stdout[-1000:] + out.stderr[-3000:]
