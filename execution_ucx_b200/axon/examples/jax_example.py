"""Arrays of another library through the RPC runtime (the counterpart of the reference's jax_example.py and
jax_cuda_example.py). The runtime needs nothing of an array type but the DLPack protocol: ``__dlpack__`` and
``__dlpack_device__`` to send it, and a ``from_dlpack_fn`` to get results back as that type. With JAX installed
the example uses ``jax.Array``; without it, a twenty-line array class that offers exactly that protocol and
nothing else, which shows how little it takes.

    python -m execution_ucx_b200.axon.examples.jax_example
"""
import asyncio

import numpy


class DLPackOnlyArray:
    """The least an array type has to offer: the two DLPack methods, and a constructor from anything that has them."""

    def __init__(self, values):
        self._a = numpy.ascontiguousarray(values)

    def __dlpack__(self, stream=None, **kwargs):
        return self._a.__dlpack__()

    def __dlpack_device__(self):
        return self._a.__dlpack_device__()

    @classmethod
    def from_dlpack(cls, other):
        return cls(numpy.from_dlpack(other))

    def __mul__(self, k):
        return DLPackOnlyArray(self._a * k)

    def tolist(self):
        return self._a.tolist()


def _array_library():
    """(array type, from_dlpack, arange) of JAX when it is installed, else of the stand-in above."""
    try:
        import jax
        import jax.numpy as jnp
        return "jax", jax.Array, jnp.from_dlpack, lambda n: jnp.arange(float(n))
    except ImportError:
        return "a DLPack-only array type", DLPackOnlyArray, DLPackOnlyArray.from_dlpack, lambda n: DLPackOnlyArray(numpy.arange(float(n)))


async def main() -> None:
    from execution_ucx_b200 import axon
    name, Array, from_dlpack, arange = _array_library()
    server = axon.AxonRuntime("jax_server", timeout=5000)
    client = axon.AxonRuntime("jax_client", timeout=5000)

    async def double(x: Array) -> Array:
        return x * 2

    server.register_function(double, from_dlpack_fn=from_dlpack)
    server.start_server()
    client.start_client()
    await client.connect_endpoint_async(server.get_local_address(), "jax_server")
    y = await client.invoke(arange(8), worker_name="jax_server", session_id=1, function="double", from_dlpack_fn=from_dlpack)
    assert isinstance(y, Array)
    print(f"double (arrays: {name}):", y.tolist())
    client.stop()
    server.stop()


if __name__ == "__main__":
    asyncio.run(main())
