"""Child program of tests/test_services_gpu.py: run under torch.distributed.run with one process per GPU.

Every rank starts one runtime, connects to every other rank's, and then checks, through the runtime's
own API: the echo RPC (eager, pulled and pushed sizes), the remote GEMM served by the partner in the three
operand formats against fp32 references, the all-peers remote GEMM, and MoE dispatch + combine on buffers
whose handles were exchanged by Axon calls."""
import asyncio
import os
import sys
from pathlib import Path

sys.path.insert(0, str(Path(__file__).resolve().parent.parent))

import torch
import torch.distributed as dist


async def main():
    from execution_ucx_b200.models.workloads import AxonTensorRpc, MoeAxon, RemoteGemmAxon
    from execution_ucx_b200.parallel.peer import PeerGroup
    rank, world = dist.get_rank(), dist.get_world_size()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    group = PeerGroup(rank, world, dev)
    api = AxonTensorRpc(group, timeout_ms=30000)
    await api.start(connect_all=True)
    # echo at eager sizes (one slot of the peer's ring, a run of slots) and at a pushed size
    for n in (2048, 1 << 21, 1 << 24):
        x = torch.randn(n // 2, device=dev).to(torch.bfloat16)
        y = await api.step(x)
        assert torch.equal(y.view(torch.int16), x.view(torch.int16)), f"echo of {n} bytes differs"
        del y
    st = api.transport_stats()
    assert st["device_staged"] == 0 and st["device_eager_sent"] >= 2 and st["device_pushes"] >= 1, st
    await api.barrier()
    # remote GEMM served by the partner, each operand format
    for fmt, tol in (("bf16", 3e-2), ("fp8_block", 3e-2), ("mxfp8", 3e-2)):
        w = RemoteGemmAxon(api, 512, 768, 1024, fmt=fmt)
        await api.barrier()
        for _ in range(2):
            await w.step()
        err = w.max_abs_err(256)
        assert err < tol * 8, f"remote gemm {fmt}: max abs err {err}"
        await api.barrier()
    # every rank calls every other rank's weight at once
    w = RemoteGemmAxon(api, 512, 512, 1024, fmt="bf16", peers="all", weight_id=11)
    await api.barrier()
    await w.step()
    assert w.max_abs_err(256) < 0.25
    await api.barrier()
    assert api.server.gemm_launches() >= 6 + (world - 1)
    # MoE on runtime-exchanged buffers
    for fp8 in (False, True):
        m = await MoeAxon.create(api, n_tokens=256, hidden=1024, topk=4, n_experts=8 * world, fp8=fp8)
        for _ in range(2):
            out = m.step()
        torch.cuda.synchronize()
        m.a2a.check_status()
        torch.testing.assert_close(out.float(), m.reference(), rtol=2e-2, atol=2e-2)
        await m.close()
    await api.barrier()
    api.stop()
    if rank == 0:
        print("SERVICES_OK", flush=True)


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        asyncio.run(main())
    finally:
        dist.destroy_process_group()
