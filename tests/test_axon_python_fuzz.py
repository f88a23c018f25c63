"""Randomised calls through the Python API: whatever goes in as an argument comes back unchanged from a function
that returns its arguments (values of every wire type, lists, nested lists, tensors of every rank and type).
The fixed cases below are what such runs have found."""
import asyncio

import numpy as np
import pytest
from typing import List, Tuple

hypothesis = pytest.importorskip("hypothesis")
from hypothesis import HealthCheck, given, settings, strategies as st  # noqa: E402


@pytest.fixture(scope="module")
def axon(native_build):
    from execution_ucx_b200 import axon as ax
    return ax


@pytest.fixture(scope="module")
def call(axon):
    loop = asyncio.new_event_loop()
    state = {}

    async def setup():
        server = axon.AxonRuntime("fuzz_srv", timeout=5000)
        client = axon.AxonRuntime("fuzz_cli", timeout=5000)

        async def prims(a: int, b: float, c: str, d: bool) -> Tuple[int, float, str, bool]:
            return a, b, c, d

        async def lists(xs: List[int], ys: List[float], zs: List[bool], ss: List[str]) -> Tuple[List[int], List[float], List[bool], List[str]]:
            return xs, ys, zs, ss

        async def nested(n: List[List[int]], m: List[List[float]], b: List[List[bool]]) -> Tuple[List[List[int]], List[List[float]], List[List[bool]]]:
            return n, m, b

        async def tensors(x: np.ndarray, k: int, xs: List[np.ndarray]) -> Tuple[int, np.ndarray, List[np.ndarray]]:
            return k, x, xs

        async def one(x: np.ndarray) -> np.ndarray:
            return x

        for f in (prims, lists, nested, tensors, one):
            server.register_function(f, from_dlpack_fn=np.from_dlpack)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "fuzz_srv")
        state["server"], state["client"] = server, client

    asyncio.set_event_loop(loop)
    loop.run_until_complete(setup())

    def invoke(name, *args):
        return loop.run_until_complete(state["client"].invoke(*args, worker_name="fuzz_srv", session_id=1, function=name,
                                                              from_dlpack_fn=np.from_dlpack))

    yield invoke
    state["client"].stop()
    state["server"].stop()
    loop.close()


ints = st.integers(min_value=-(2 ** 63), max_value=2 ** 63 - 1)
floats = st.floats(allow_nan=False)
texts = st.text(max_size=30)
quick = settings(max_examples=60, deadline=None, suppress_health_check=list(HealthCheck))


def test_header_params_survive_the_wire_image(axon):
    value = st.one_of(st.booleans(), ints, floats, st.text(max_size=40), st.binary(max_size=40), st.lists(ints, min_size=1, max_size=20),
                      st.lists(floats, min_size=1, max_size=20), st.lists(st.booleans(), min_size=1, max_size=20), st.none())

    @settings(max_examples=200, deadline=None)
    @given(st.lists(value, max_size=8), st.integers(0, 2 ** 32 - 1), st.integers(0, 2 ** 32 - 1))
    def check(vals, sid, fid):
        h = axon.RpcRequestHeader()
        h.session_id, h.function_id = sid, fid
        for v in vals:
            h.AddParam(v)
        back = axon.RpcRequestHeader.deserialize(h.serialize())
        assert back.session_id == sid and back.function_id == fid
        got = back.params
        assert len(got) == len(vals)
        for v, g in zip(vals, got):
            if isinstance(v, bytes):
                assert (g.encode() if isinstance(g, str) else bytes(g)) == v
            else:
                assert g == v
        # the same values as the results of a response
        r = axon.RpcResponseHeader()
        r.session_id = sid
        for v in vals:
            r.AddResult(v)
        rback = axon.RpcResponseHeader.deserialize(r.serialize())
        assert rback.session_id == sid and rback.ok and len(rback.results) == len(vals)
        for v, g in zip(vals, rback.results):
            if isinstance(v, bytes):
                assert (g.encode() if isinstance(g, str) else bytes(g)) == v
            else:
                assert g == v

    check()


def test_values_of_every_kind_come_back(call):
    @quick
    @given(ints, floats, texts, st.booleans())
    def prims(a, b, c, d):
        r = call("prims", a, b, c, d)
        assert r == (a, b, c, d) and type(r[0]) is int and type(r[3]) is bool

    @quick
    @given(st.lists(ints, min_size=1, max_size=10), st.lists(floats, min_size=1, max_size=10), st.lists(st.booleans(), min_size=1, max_size=10),
           st.lists(texts, min_size=1, max_size=6))
    def lists(xs, ys, zs, ss):
        assert call("lists", xs, ys, zs, ss) == (xs, ys, zs, ss)

    def nl(e):
        return st.lists(st.lists(e, max_size=5), min_size=1, max_size=5)

    @quick
    @given(nl(ints), nl(floats), nl(st.booleans()))
    def nested(n, m, b):
        assert call("nested", n, m, b) == (n, m, b)

    prims()
    lists()
    nested()


def test_tensors_of_every_rank_and_type_come_back(call):
    shapes = st.lists(st.integers(0, 5), min_size=0, max_size=3)
    dtypes = st.sampled_from([np.float32, np.float64, np.int32, np.int64, np.uint8, np.int16, np.float16, np.bool_])

    @quick
    @given(shapes, dtypes, st.integers(-5, 5), st.lists(st.tuples(shapes, dtypes), min_size=1, max_size=4), st.integers(0, 2 ** 31))
    def tensors(shape, dtype, k, others, seed):
        rng = np.random.default_rng(seed)

        def make(s, d):
            return np.asarray(np.asarray(rng.random(s) * 100).astype(d))

        x, xs = make(shape, dtype), [make(s, d) for s, d in others]
        r = call("tensors", x, k, xs)
        assert r[0] == k and len(r) == 2 + len(xs)
        for want, got in zip([x] + xs, r[1:]):
            assert got.dtype == want.dtype and got.shape == want.shape and np.array_equal(got, want)

    tensors()


def test_cases_that_randomised_runs_found(call):
    # a list of strings whose blob is shorter than 16 bytes and holds NULs (the wire image's short string form ends at a NUL)
    assert call("lists", [1], [1.0], [True], ["a", "b"]) == ([1], [1.0], [True], ["a", "b"])
    assert call("prims", 0, 0.0, "nul\x00inside", False)[2] == "nul\x00inside"
    # a tensor without elements travels as no payload at all and is made on arrival
    for shape in ((0,), (2, 0, 3)):
        got = call("one", np.zeros(shape, np.float32))
        assert got.shape == shape and got.dtype == np.float32
    # a rank-0 tensor is one element on the wire, alone and among others
    assert float(call("one", np.asarray(np.float32(3.0)))) == 3.0
    r = call("tensors", np.asarray(np.float64(2.5)), 1, [np.ones((1,), np.float32), np.asarray(np.int16(7))])
    assert r[1].shape == () and float(r[1]) == 2.5 and r[2].shape == (1,) and r[3].shape == () and int(r[3]) == 7
    r = call("tensors", np.zeros((0,), np.float32), 4, [np.zeros((0, 3), np.int64), np.ones((2,), np.float32)])
    assert r[0] == 4 and r[1].shape == (0,) and r[2].shape == (0, 3) and r[2].dtype == np.int64 and r[3].tolist() == [1.0, 1.0]


def test_empty_and_rank0_torch_tensors(axon):
    torch = pytest.importorskip("torch")

    async def main():
        server = axon.AxonRuntime("fuzz_t_srv", timeout=5000)
        client = axon.AxonRuntime("fuzz_t_cli", timeout=5000)

        async def echo(x: torch.Tensor) -> torch.Tensor:
            return x

        async def both(x: torch.Tensor, ys: List[torch.Tensor]) -> List[torch.Tensor]:
            return [x] + ys

        server.register_function(echo)
        server.register_function(both)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "fuzz_t_srv")
        for x in (torch.zeros(0), torch.zeros(3, 0, dtype=torch.bfloat16), torch.tensor(2.5), torch.tensor(7, dtype=torch.int64),
                  torch.tensor(1.5, dtype=torch.bfloat16), torch.arange(6, dtype=torch.int32).reshape(2, 3)):
            y = await client.invoke(x, worker_name="fuzz_t_srv", session_id=1, function="echo")
            assert isinstance(y, torch.Tensor) and y.dtype == x.dtype and y.shape == x.shape and torch.equal(y, x), (x, y)
        out = await client.invoke(torch.tensor(4.0), [torch.zeros(0, 2), torch.ones(2), torch.tensor(3, dtype=torch.int16)],
                                  worker_name="fuzz_t_srv", session_id=1, function="both")
        assert [tuple(t.shape) for t in out] == [(), (0, 2), (2,), ()] and float(out[0]) == 4.0 and int(out[3]) == 3
        client.stop()
        server.stop()

    loop = asyncio.new_event_loop()
    try:
        asyncio.set_event_loop(loop)
        loop.run_until_complete(main())
    finally:
        loop.close()
