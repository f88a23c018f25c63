"""Python API of the runtime: two AxonRuntime objects (server + client) over loopback in one process."""
import asyncio

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


def test_types_and_param_inference(axon):
    h = axon.RpcRequestHeader()
    h.session_id, h.function_id = 5, 9
    for v in (True, 7, 2.5, "text", b"\x00\x01", [1, 2, 3], [1.0, 2], [True, False], None):
        h.AddParam(v)
    kinds = [t for t, _, _ in h.params_meta]
    P = axon.ParamType
    assert kinds == [P.PRIMITIVE_BOOL, P.PRIMITIVE_INT64, P.PRIMITIVE_FLOAT64, P.STRING, P.VECTOR_UINT8, P.VECTOR_INT64,
                     P.VECTOR_FLOAT64, P.VECTOR_BOOL, P.VOID]
    back = axon.RpcRequestHeader.deserialize(h.serialize())
    assert back.params == [True, 7, 2.5, "text", b"\x00\x01", [1, 2, 3], [1.0, 2.0], [True, False], None]
    assert axon.RpcResponseHeader().status == {"value": 0, "category_name": ""} or axon.RpcResponseHeader().status["value"] == 0
    assert axon.PayloadType.MONOSTATE == axon.PayloadType.NO_PAYLOAD
    assert back.session_id == 5 and back.function_id == 9
    m = axon.TensorMeta.from_tensor(np.zeros((3, 4), dtype=np.float32))
    assert m.shape == [3, 4] and m.dtype.bits == 32 and m.nbytes() == 48
    with pytest.raises(ValueError):
        axon.TensorMeta.from_tensor(np.zeros((4, 4))[:, ::2])
    assert axon.function_id_from_name("f", "w") == axon.function_id_from_name("f", "w") != axon.function_id_from_name("g", "w")
    assert isinstance(axon.auto_detect(), axon.Device) and str(axon.cuda(1)) == "cuda:1"


def test_invoke_numpy_eager_and_rendezvous(axon):
    async def main():
        server = axon.AxonRuntime("py_server", timeout=5000)
        client = axon.AxonRuntime("py_client", timeout=5000)

        async def add_scaled(x: np.ndarray, k: int, bias: float) -> np.ndarray:
            return x * k + bias

        async def stats(xs: List[np.ndarray], tag: str) -> Tuple[str, float, List[int]]:
            return tag + "!", float(sum(a.sum() for a in xs)), [a.size for a in xs]

        async def boom(n: int) -> int:
            raise ValueError("bad input %d" % n)

        server.register_function(add_scaled)
        server.register_function(stats)
        server.register_function(boom)
        server.start_server()
        client.start_client()
        conn = await client.connect_endpoint_async(server.get_local_address(), "py_server")
        assert conn != 0
        sigs = axon.deserialize_signatures(server.get_local_signatures())
        assert sorted(s.function_name for s in sigs) == ["add_scaled", "boom", "stats"]
        for n in (16, 200_000):  # small (inline) and large (rendezvous) payloads
            x = np.arange(n, dtype=np.float32)
            y = await client.invoke(x, 3, 0.5, worker_name="py_server", session_id=1, function="add_scaled")
            assert isinstance(y, np.ndarray) and y.dtype == np.float32
            np.testing.assert_array_equal(y, x * 3 + 0.5)
        a, b = np.ones(10, dtype=np.float64), np.full(50_000, 2.0)
        tag, total, sizes = await client.invoke([a, b], "t", worker_name="py_server", session_id=1, function="stats")
        assert tag == "t!" and total == 10 + 100_000 and sizes == [10, 50_000]
        with pytest.raises(RuntimeError) as e:
            await client.invoke(4, worker_name="py_server", session_id=2, function="boom")
        assert "bad input 4" in str(e.value) and "(session_id: 2)" in str(e.value)
        with pytest.raises(RuntimeError):
            await client.invoke(1, worker_name="py_server", session_id=2, function="missing_function")
        client.stop()
        server.stop()

    from typing import List, Tuple  # noqa: F401  (used by the annotations above)
    globals().update(List=List, Tuple=Tuple)
    run(main())


def test_memory_policy_returns_the_same_object(axon):
    async def main():
        server = axon.AxonRuntime("mp_server", timeout=5000)
        client = axon.AxonRuntime("mp_client", timeout=5000)

        async def double(x: np.ndarray) -> np.ndarray:
            return x * 2

        server.register_function(double)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "mp_server")
        made = []

        def policy(metas):
            t = np.empty(metas[0].shape, dtype=np.float32)
            made.append(t)
            return t

        x = np.arange(100_000, dtype=np.float32)
        y = await client.invoke(x, worker_name="mp_server", session_id=1, function="double", memory_policy=policy)
        assert len(made) == 1 and y is made[0]          # the rendezvous path fills the policy's tensor
        np.testing.assert_array_equal(y, x * 2)
        small = await client.invoke(x[:8].copy(), worker_name="mp_server", session_id=1, function="double", memory_policy=policy)
        assert len(made) == 1                            # small results do not consult the policy
        np.testing.assert_array_equal(small, x[:8] * 2)
        client.stop()
        server.stop()

    run(main())


def test_raw_api_retention_and_checkpoint(axon, tmp_path):
    async def main():
        server = axon.AxonRuntime("raw_server", timeout=5000)
        client = axon.AxonRuntime("raw_client", timeout=5000)
        seen = []

        async def handler(values):          # raw functions get their parameters as plain positional values
            seen.append(list(values))
            return sum(values)

        P = axon.ParamType
        server.register_function_raw(77, "sum", [P.VECTOR_INT64], [P.PRIMITIVE_INT64], axon.PayloadType.NO_PAYLOAD,
                                     axon.PayloadType.NO_PAYLOAD, handler, None, lambda header, msg_id: True)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "raw_server")
        h = axon.RpcRequestHeader()
        h.session_id, h.function_id = 3, 77
        h.AddParam([1, 2, 3, 4])
        assert await client.invoke_raw("raw_server", h) == 10
        assert seen == [[1, 2, 3, 4]]
        assert server.stored_request_count() == 1       # the retention policy kept the request
        path = server.save_stored_requests(str(tmp_path), "keep")
        assert path.endswith(".avro")
        assert await server.process_stored_requests() == 1 and len(seen) == 2
        other = axon.AxonRuntime("restore", timeout=1000)
        assert other.load_stored_requests(path) == 1 and other.stored_request_count() == 1
        client.stop()
        server.stop()

    run(main())


def test_wire_dtype_converts_host_tensors_before_they_are_sent(axon):
    """``wire_dtype``: floating-point tensors travel in another type than they have in memory. On the host the
    conversion happens before the send (on a GPU the transfer kernel does it on the way); what the function sees,
    and what comes back, has the wire type."""
    torch = pytest.importorskip("torch")

    async def main():
        server = axon.AxonRuntime("wd_server", timeout=5000)
        client = axon.AxonRuntime("wd_client", timeout=5000)
        seen = []

        async def what_arrived(x: torch.Tensor) -> torch.Tensor:
            seen.append(x.dtype)
            return x

        async def halves(xs: List[np.ndarray]) -> List[np.ndarray]:
            seen.append([a.dtype for a in xs])
            return xs

        async def as_float(x: torch.Tensor) -> torch.Tensor:
            return x.float() * 3.0

        server.register_function(what_arrived)
        server.register_function(halves)
        server.register_function(as_float, wire_dtype=torch.float16)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "wd_server")
        for n in (100, 100000):       # eager and rendezvous
            x = torch.randn(n)
            y = await client.invoke(x, worker_name="wd_server", session_id=1, function="what_arrived", wire_dtype=torch.bfloat16)
            assert seen[-1] == torch.bfloat16 and y.dtype == torch.bfloat16
            assert torch.equal(y, x.to(torch.bfloat16))
        ys = await client.invoke([np.ones(8, dtype=np.float32), np.arange(4, dtype=np.float64)], worker_name="wd_server", session_id=1,
                                 function="halves", wire_dtype=np.float16, from_dlpack_fn=np.from_dlpack)
        assert seen[-1] == [np.dtype("float16"), np.dtype("float16")]
        assert [a.dtype for a in ys] == [np.dtype("float16")] * 2 and float(ys[1][3]) == 3.0
        z = await client.invoke(torch.ones(16, dtype=torch.float64), worker_name="wd_server", session_id=1, function="as_float")
        assert z.dtype == torch.float16 and float(z[0]) == 3.0      # the function's fp32 result came back as fp16
        with pytest.raises(ValueError):
            client.invoke(np.ones(4, dtype=np.float32), worker_name="wd_server", session_id=1, function="what_arrived", wire_dtype=torch.bfloat16)
        with pytest.raises(ValueError):
            client.invoke(torch.ones(4), worker_name="wd_server", session_id=1, function="what_arrived", wire_dtype=torch.int32)
        client.stop()
        server.stop()

    run(main())


def test_native_call_conversion_agrees_with_the_python_layer(axon, monkeypatch):
    """Arguments and results are drawn from a message by native code where it covers the case and by the
    Python layer otherwise: both must give the same values for every shape of call."""
    from typing import List, Tuple

    import torch

    async def battery(tag: str):
        server = axon.AxonRuntime("conv_srv_" + tag, timeout=5000)
        client = axon.AxonRuntime("conv_cli_" + tag, timeout=5000)

        async def mixed(a: int, x: np.ndarray, s: str, f: float, flags: List[bool]) -> Tuple[int, np.ndarray, str]:
            return a + len(flags), x * f, s.upper()

        async def many(xs: List[np.ndarray], k: int) -> List[np.ndarray]:
            return [x + k for x in xs]

        async def nested(groups: List[List[np.ndarray]], names: List[str], table: List[List[int]]) -> Tuple[List[int], float]:
            return [len(g) for g in groups] + [len(names), sum(map(sum, table))], float(sum(float(t.sum()) for g in groups for t in g))

        async def flat_from_nested(xs: List[np.ndarray]) -> int:
            return len(xs)

        async def nothing() -> None:
            return None

        async def plain(a: int, b: float) -> float:
            return a * b

        async def torch_echo(x: torch.Tensor) -> torch.Tensor:
            return x

        async def pair(a: int, b: str) -> Tuple[int, str]:
            return a, b

        for fn in (mixed, many, nested, flat_from_nested, nothing, plain, pair):
            server.register_function(fn, from_dlpack_fn=np.from_dlpack)
        server.register_function(torch_echo)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "conv_srv_" + tag)
        call = lambda name, *a, **k: client.invoke(*a, worker_name="conv_srv_" + tag, session_id=1, function=name,  # noqa: E731
                                                   from_dlpack_fn=k.get("fd", np.from_dlpack))
        x = np.arange(12, dtype=np.float32).reshape(3, 4)
        big = np.arange(1 << 16, dtype=np.float32)             # rendezvous: the response lands through the memory policy path
        out = {}
        out["mixed"] = await call("mixed", 5, x, "abc", 0.5, [True, False, True])
        out["mixed_big"] = await call("mixed", 1, big, "q", 2.0, [False])
        out["many"] = await call("many", [x, x[:1].copy(), big], 3)
        out["nested"] = await call("nested", [[x, x], [], [x]], ["a", "b"], [[1, 2], [3]])
        out["flat_from_nested"] = await call("flat_from_nested", [[x], [x, x]])
        out["nothing"] = await call("nothing")
        out["plain"] = await call("plain", 6, 1.5)
        out["pair"] = await call("pair", 7, "seven")
        out["torch"] = await call("torch_echo", torch.arange(10, dtype=torch.int32), fd=None)
        with pytest.raises(RuntimeError) as too_few:
            await call("mixed", 5, "abc")
        out["error"] = str(too_few.value).split(" (function_id")[0]   # the id hashes the worker's name, which differs between the two runs
        client.stop()
        server.stop()
        return out

    def normal(v):
        if isinstance(v, (tuple, list)):
            return type(v).__name__, [normal(x) for x in v]
        if isinstance(v, np.ndarray):
            return "ndarray", str(v.dtype), v.shape, v.tobytes()
        if hasattr(v, "numpy"):
            return "torch", str(v.dtype), tuple(v.shape), v.numpy().tobytes()
        return v

    native = run(battery("n"))
    calls = {"plan": 0, "results": 0}

    class PythonOnlyPlan:
        def __init__(self, *a, **k):
            pass

        def args(self, header, payload):
            calls["plan"] += 1
            return NotImplemented

    def python_only_results(*a):
        calls["results"] += 1
        return NotImplemented

    monkeypatch.setattr(axon._axon, "_ArgPlan", PythonOnlyPlan)
    monkeypatch.setattr(axon._axon, "_results_to_python", python_only_results)
    python = run(battery("p"))
    assert calls["plan"] >= 9 and calls["results"] >= 9
    assert native.keys() == python.keys()
    for key in native:
        assert normal(native[key]) == normal(python[key]), key
    assert native["mixed"][0] == 8 and native["mixed"][1] == "ABC" and native["mixed"][2].shape == (3, 4) and native["nothing"] is None and native["plain"] == 9.0
    assert native["nested"][0] == [2, 0, 1, 2, 6] and native["flat_from_nested"] == 3 and native["pair"] == (7, "seven")


def test_a_handler_that_breaks_its_annotation_fails_the_call(axon):
    async def main():
        server = axon.AxonRuntime("brk_srv", timeout=3000)
        client = axon.AxonRuntime("brk_cli", timeout=3000)

        async def nothing_for_a_tensor(x: np.ndarray) -> np.ndarray:
            return None

        async def number_for_a_tensor(x: np.ndarray) -> np.ndarray:
            return 5

        async def fine(x: np.ndarray) -> np.ndarray:
            return x

        for f in (nothing_for_a_tensor, number_for_a_tensor, fine):
            server.register_function(f, from_dlpack_fn=np.from_dlpack)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "brk_srv")
        x = np.arange(4, dtype=np.float32)
        for name, text in (("nothing_for_a_tensor", "returned None"), ("number_for_a_tensor", "__dlpack__")):
            with pytest.raises(RuntimeError, match=text):
                await client.invoke(x, worker_name="brk_srv", session_id=1, function=name, from_dlpack_fn=np.from_dlpack)
        assert np.array_equal(await client.invoke(x, worker_name="brk_srv", session_id=1, function="fine", from_dlpack_fn=np.from_dlpack), x)
        client.stop()
        server.stop()

    run(main())
