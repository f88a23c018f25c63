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
    for n in (2048, 1 << 21, 1 << 25):
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
    await mixed_traffic(api, dev, rank, world)
    await api.barrier()
    api.stop()
    if rank == 0:
        print("SERVICES_OK", flush=True)


async def mixed_traffic(api, dev, rank, world):
    """Every rank serves and calls at once: 150 calls of random size (dense, strided, converted) to random peers,
    16 in flight, every reply checked. Ring slots, pushes in both directions and the descriptor of every peer
    are all in use together."""
    import random
    table = {(2, 32): torch.float32, (2, 16): torch.float16, (4, 16): torch.bfloat16}

    def fresh(metas):
        m = metas[0]
        return torch.empty(m.shape, dtype=table[(m.dtype.code, m.dtype.bits)], device=dev)

    async def twice(x: torch.Tensor) -> torch.Tensor:
        return x * 2.0

    api.server.register_function(twice, memory_policy=fresh)
    await api.barrier()
    rng = random.Random(1000 + rank)
    sem = asyncio.Semaphore(16)
    failures = []
    peers = [n for i, n in enumerate(api.names) if i != rank]

    async def one(i):
        async with sem:
            kind = rng.choice(("dense", "dense", "strided", "cast"))
            n = int(2 ** rng.uniform(6, 22))
            wire = None
            if kind == "strided":
                rows = max(2, int(n ** 0.5))
                x = torch.randn(rows, rows + 3, device=dev)[:, 1:-2].t()
            else:
                x = torch.randn(n, device=dev)
                if kind == "cast":
                    wire = torch.bfloat16
            y = await api.client.invoke(x, worker_name=rng.choice(peers), session_id=i, function="twice", memory_policy=fresh, wire_dtype=wire)
            ref = x.contiguous().to(wire or torch.float32) * 2.0
            if y.dtype != ref.dtype or y.shape != x.shape or not torch.equal(y, ref):
                failures.append((i, kind, tuple(x.shape), str(y.dtype)))

    await asyncio.gather(*[one(i) for i in range(150)])
    assert not failures, f"rank {rank}: {failures[:5]}"
    st = api.transport_stats()
    assert st["device_staged"] == 0 and st["device_packs"] == 0, st


if __name__ == "__main__":
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    try:
        asyncio.run(main())
    finally:
        dist.destroy_process_group()
