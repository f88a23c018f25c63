"""One tiny pass over each data-plane path (used by the smoke entry point)."""
from __future__ import annotations

import torch


def run(device: torch.device) -> None:
    from ..ops import moe, tensor_xfer as tx
    torch.cuda.set_device(device)
    # tensor RPC data plane: pack + cast + "+1.0" handler + flag
    src = torch.rand(3, 1000, device=device).t()
    dst = torch.zeros(3000, dtype=torch.bfloat16, device=device)
    flag = torch.zeros(1, dtype=torch.int64, device=device)
    tx.push(src, dst, op=tx.OP_ADD, op_arg=1.0, flag_ptr=flag.data_ptr(), flag_value=1)
    torch.cuda.synchronize()
    assert int(flag.item()) == 1
    assert torch.equal(dst.float(), (src.contiguous().view(-1) + 1.0).to(torch.bfloat16).float())
    # MoE dispatch -> identity expert -> combine, 2 logical ranks
    ranks = moe.MoeAllToAll.emulated(2, 32, 256, 2, 8)
    xs = [torch.randn(32, 256, device=device).to(torch.bfloat16) for _ in ranks]
    idx = [torch.rand(32, 8, device=device).topk(2, -1).indices.to(torch.int32) for _ in ranks]
    w = [torch.softmax(torch.randn(32, 2, device=device), -1) for _ in ranks]
    for r, m in enumerate(ranks):
        m.dispatch(xs[r], idx[r], w[r])
    for m in ranks:
        m.expert_ready()
    for r, m in enumerate(ranks):
        out = m.combine()
        torch.cuda.synchronize()
        m.check_status()
        ref = moe.reference_dispatch_combine(xs[r], idx[r], w[r], False)
        torch.testing.assert_close(out.float(), ref, rtol=2e-2, atol=2e-2)
    try:
        from ..ops import remote_gemm
    except ImportError:
        remote_gemm = None
    if remote_gemm is not None:
        remote_gemm.smoke(device)
    _axon_round_trip(device)


def _axon_round_trip(device: torch.device) -> None:
    """One RPC with a device tensor through the runtime and its Python binding."""
    import asyncio

    from .. import axon

    async def main():
        index = device.index or 0
        server = axon.AxonRuntime("smoke_server", timeout=10000, device=axon.cuda(index))
        client = axon.AxonRuntime("smoke_client", timeout=10000, device=axon.cuda(index))

        async def add_one(x: torch.Tensor) -> torch.Tensor:
            return x + 1.0

        policy = lambda metas: torch.empty(metas[0].shape, dtype=torch.float32, device=device)  # noqa: E731
        server.register_function(add_one, memory_policy=policy)
        server.start_server()
        client.start_client()
        await client.connect_endpoint_async(server.get_local_address(), "smoke_server")
        x = torch.rand(1 << 16, device=device)
        y = await client.invoke(x, worker_name="smoke_server", session_id=1, function="add_one", memory_policy=policy)
        assert y.is_cuda and torch.equal(y, x + 1.0)
        client.stop()
        server.stop()

    asyncio.run(main())
