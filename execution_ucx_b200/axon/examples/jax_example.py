"""JAX arrays through the RPC runtime (the counterpart of the reference's jax_example.py and
jax_cuda_example.py). Any array type that speaks DLPack works: pass ``from_dlpack_fn`` when the
result should come back as a type other than the one that was sent.

    python -m execution_ucx_b200.axon.examples.jax_example
"""
from __future__ import annotations

import asyncio


async def main() -> None:
    try:
        import jax
        import jax.numpy as jnp
    except ImportError:
        print("jax is not installed here; the same calls work with numpy arrays or torch tensors "
              "(see pytorch_example.py)")
        return
    from execution_ucx_b200 import axon
    server = axon.AxonRuntime("jax_server", timeout=5000)
    client = axon.AxonRuntime("jax_client", timeout=5000)

    async def double(x: jax.Array) -> jax.Array:
        return x * 2

    server.register_function(double, from_dlpack_fn=jnp.from_dlpack)
    server.start_server()
    client.start_client()
    await client.connect_endpoint_async(server.get_local_address(), "jax_server")
    y = await client.invoke(jnp.arange(8.0), worker_name="jax_server", session_id=1, function="double",
                            from_dlpack_fn=jnp.from_dlpack)
    print("double:", y)
    client.stop()
    server.stop()


if __name__ == "__main__":
    asyncio.run(main())
