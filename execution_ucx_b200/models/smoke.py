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
    # the same with e4m3 rows and per-128 scales (the fp8 dispatch and combine kernels)
    ranks8 = moe.MoeAllToAll.emulated(2, 32, 256, 2, 8, fp8=True)
    for r, m in enumerate(ranks8):
        m.dispatch(xs[r], idx[r], w[r])
    for m in ranks8:
        m.expert_ready()
    for r, m in enumerate(ranks8):
        out = m.combine()
        torch.cuda.synchronize()
        m.check_status()
        torch.testing.assert_close(out.float(), moe.reference_dispatch_combine(xs[r], idx[r], w[r], True), rtol=2e-2, atol=2e-2)
    from ..ops import remote_gemm
    remote_gemm.smoke(device)
    _fp8_block_gemm(device)
    _data_plane_echo_and_pingpong(device)
    _axon_round_trip(device)


def _fp8_block_gemm(device: torch.device) -> None:
    """The e4m3 GEMM with fp32 block scales (1x128 on X, 128x128 on W)."""
    from ..ops import remote_gemm as g
    x = torch.randn(256, 512, device=device).to(torch.bfloat16)
    w = (torch.randn(512, 512, device=device) * 0.05).to(torch.bfloat16)
    gemm = g.RemoteGemmFp8(w, 256)
    xq, xs = g.quantize_rows_1x128(x)
    y = torch.zeros(256, 512, dtype=torch.bfloat16, device=device)
    gemm(xq.data_ptr(), xs.data_ptr(), 256, y.data_ptr(), x_is_local=True)
    torch.cuda.synchronize()
    gemm.check_status()
    torch.testing.assert_close(y.float(), g.dequantized_reference(xq, xs, gemm.w_q_t, gemm.w_scale), rtol=3e-2, atol=3e-2)


def _data_plane_echo_and_pingpong(device: torch.device) -> None:
    """The one-launch echo step (request, handler, response as phases of one kernel), a plain byte copy
    through the transfer kernel, and the device-driven ping-pong, all as a loopback on this GPU."""
    from ..models.workloads import DevicePingPong, TensorRpcEcho
    from ..ops import tensor_xfer as tx
    from ..parallel.peer import PeerGroup
    group = PeerGroup(0, 1, device)
    n = 1 << 20
    src = torch.randn(n // 2, device=device).to(torch.bfloat16)
    rpc = TensorRpcEcho(group, n)
    resp = rpc.step(src)
    torch.cuda.synchronize()
    rpc.check_status()
    assert torch.equal(resp.view(torch.int16), src.view(torch.int16))
    rpc.close()
    raw = torch.randint(0, 255, (n + 5,), dtype=torch.uint8, device=device)
    out = torch.zeros_like(raw)
    tx.push(raw, out)
    torch.cuda.synchronize()
    assert torch.equal(raw, out)
    pp = DevicePingPong(group, 1 << 16)
    rtt = pp.run(1 << 16, 4)
    assert rtt.numel() == 4 and int(rtt.min()) > 0
    pp.close()


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
        # 1 KiB and 256 KiB travel eagerly into the receive ring (one CTA of a batched launch; a launch of
        # several CTAs), 32 MiB is pushed by the sender's kernel
        for n in (256, 1 << 16, 1 << 23):
            x = torch.rand(n, device=device)
            y = await client.invoke(x, worker_name="smoke_server", session_id=1, function="add_one", memory_policy=policy)
            assert y.is_cuda and torch.equal(y, x + 1.0)
            del y
        # a transposed 32 MiB matrix is gathered out of the sender's memory by the receiver's pull
        xt = torch.rand(4096, 2048, device=device).t()
        y = await client.invoke(xt, worker_name="smoke_server", session_id=1, function="add_one", memory_policy=policy)
        assert torch.equal(y, xt.contiguous() + 1.0)
        del y
        # the remote GEMM as an Axon function of the server, called by the client
        w = (torch.randn(256, 512, device=device) * 0.05).to(torch.bfloat16)
        server.serve_gemm(1, w, "bf16", max_m=256)
        gx = torch.randn(256, 256, device=device).to(torch.bfloat16)
        gy = torch.zeros(256, 512, dtype=torch.bfloat16, device=device)
        assert await client.remote_gemm(gx, gy, worker_name="smoke_server", weight_id=1) == 0
        torch.testing.assert_close(gy.float(), gx.float() @ w.float(), rtol=2e-2, atol=2e-2)
        client.stop()
        server.stop()

    asyncio.run(main())
