"""Library baselines for the three workloads: NCCL send/recv, cuBLAS (through torch) and NCCL
all-to-all. Nothing here uses this package's kernels; the benchmark reports these numbers beside
its own so that each fused kernel has a same-machine, same-shape comparison. They are baselines,
not part of the product's data path.

The reference has no GEMM and no all-to-all of its own; what it would run for these workloads is a
transfer followed by a library call, which is what these classes do.
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def _partner(rank: int, world: int) -> int:
    return rank ^ 1 if world > 1 else rank


class NcclEcho:
    """Echo of one tensor with the partner rank: send/recv there, send/recv back (two D2D copies on one rank)."""

    def __init__(self, rank: int, world: int, nbytes: int, device):
        self.rank, self.world, self.peer = rank, world, _partner(rank, world)
        self.req = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=device)
        self.resp = torch.empty(nbytes // 2, dtype=torch.bfloat16, device=device)

    def step(self, src: torch.Tensor) -> torch.Tensor:
        n = src.numel()
        if self.world == 1:
            self.req[:n].copy_(src)
            self.resp[:n].copy_(self.req[:n])
            return self.resp[:n]
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, src, self.peer), dist.P2POp(dist.irecv, self.req[:n], self.peer)]):
            work.wait()
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, self.req[:n], self.peer),
                                            dist.P2POp(dist.irecv, self.resp[:n], self.peer)]):
            work.wait()
        return self.resp[:n]


class RecvGemmSend:
    """Remote GEMM the library way: receive the partner's X, cuBLAS matmul, send Y back."""

    def __init__(self, rank: int, world: int, m: int, n: int, k: int, device):
        self.rank, self.world, self.peer = rank, world, _partner(rank, world)
        g = torch.Generator(device=device).manual_seed(4321 + rank)
        self.x = torch.randn(m, k, device=device, generator=g).to(torch.bfloat16)
        self.w = (torch.randn(k, n, device=device, generator=g) * 0.02).to(torch.bfloat16)
        self.x_in = torch.empty_like(self.x)
        self.y = torch.empty(m, n, dtype=torch.bfloat16, device=device)
        self.y_back = torch.empty_like(self.y)

    def step(self) -> torch.Tensor:
        if self.world == 1:
            torch.matmul(self.x, self.w, out=self.y)
            return self.y
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, self.x, self.peer), dist.P2POp(dist.irecv, self.x_in, self.peer)]):
            work.wait()
        torch.matmul(self.x_in, self.w, out=self.y)
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, self.y, self.peer), dist.P2POp(dist.irecv, self.y_back, self.peer)]):
            work.wait()
        return self.y_back


class AllToAllMoe:
    """MoE dispatch + combine with torch ops and ``all_to_all_single``: sort the (token, k) pairs by
    destination rank, exchange counts (host synchronisation), exchange rows, identity expert,
    exchange back, gate-weighted ``index_add_``."""

    def __init__(self, rank: int, world: int, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, n_experts: int):
        self.rank, self.world = rank, world
        self.x, self.idx, self.w = x, topk_idx.long(), topk_w.float()
        self.epr = n_experts // world
        t, k = self.idx.shape
        self.token_of_pair = torch.arange(t, device=x.device).repeat_interleave(k)
        self.out = torch.empty_like(x)

    def step(self) -> torch.Tensor:
        dest = (self.idx // self.epr).reshape(-1)
        order = torch.argsort(dest, stable=True)
        tok = self.token_of_pair[order]
        send_counts = torch.bincount(dest, minlength=self.world)
        if self.world == 1:
            rows = self.x[tok]                       # dispatch
            back = rows.clone()                      # expert output returns
        else:
            recv_counts = torch.empty_like(send_counts)
            dist.all_to_all_single(recv_counts, send_counts)
            sc, rc = send_counts.tolist(), recv_counts.tolist()
            rows = self.x[tok]
            recv = torch.empty(sum(rc), self.x.shape[1], dtype=self.x.dtype, device=self.x.device)
            dist.all_to_all_single(recv, rows, rc, sc)
            back = torch.empty_like(rows)
            dist.all_to_all_single(back, recv, sc, rc)
        acc = torch.zeros(self.x.shape, dtype=torch.float32, device=self.x.device)
        acc.index_add_(0, tok, back.float() * self.w.reshape(-1)[order].unsqueeze(1))
        self.out.copy_(acc)
        return self.out


class PingPongSweep:
    """Echo ping-pong at one size after another with library calls only.

    ``nccl_round_trip``: NCCL send/recv there and back (both ranks of a pair at once, as in the product's
    sweep). ``copy_engine_one_way``: ``cudaMemcpyPeerAsync`` of the same bytes into a buffer of the
    partner (mapped through CUDA IPC), both ranks at once; a round trip by the copy engine is taken as
    twice that, which leaves out whatever signalling a real protocol would need between the two legs.
    """

    def __init__(self, group, max_bytes: int):
        self.g = group
        self.rank, self.world, self.peer = group.rank, group.world, _partner(group.rank, group.world)
        dev = group.device
        self.a = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=dev)
        self.b = torch.empty(max_bytes // 2, dtype=torch.bfloat16, device=dev)
        self.inbox = group.alloc(max_bytes)      # the partner's copy of this buffer is the copy engine's target
        self.max_bytes = max_bytes

    def nccl_round_trip(self, src: torch.Tensor):
        n = src.numel()
        if self.world == 1:
            self.a[:n].copy_(src)
            self.b[:n].copy_(self.a[:n])
            return
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, src, self.peer), dist.P2POp(dist.irecv, self.a[:n], self.peer)]):
            work.wait()
        for work in dist.batch_isend_irecv([dist.P2POp(dist.isend, self.a[:n], self.peer), dist.P2POp(dist.irecv, self.b[:n], self.peer)]):
            work.wait()

    def copy_engine_one_way(self, src: torch.Tensor):
        """The driver's peer copy on the current stream; no kernel of any library touches the peer's memory."""
        import ctypes as C

        from ..ops import _native
        lib = _native.load()
        nbytes = src.numel() * src.element_size()
        peer_dev = self.peer if self.world > 1 else self.g.device.index or 0   # one process per GPU, rank == device ordinal
        _native.check(lib.eux_memcpy_peer_async(C.c_void_p(self.inbox.peer_ptrs[self.peer]), peer_dev, C.c_void_p(src.data_ptr()),
                                                self.g.device.index or 0, nbytes, C.c_void_p(torch.cuda.current_stream().cuda_stream)),
                      "cudaMemcpyPeerAsync")

    def close(self):
        self.g.free(self.inbox)


class ScaledMmBaseline:
    """fp8 GEMM the library way: ``torch._scaled_mm`` (cuBLASLt) on e4m3 operands with per-tensor scales:
    the closest library call to the block-scaled remote GEMM. Absent kernels raise, and the caller reports that."""

    def __init__(self, m: int, n: int, k: int, device):
        g = torch.Generator(device=device).manual_seed(99)
        self.x = torch.randn(m, k, device=device, generator=g).to(torch.float8_e4m3fn)
        self.w = (torch.randn(n, k, device=device, generator=g) * 0.02).to(torch.float8_e4m3fn)
        self.sx = torch.ones((), device=device)
        self.sw = torch.ones((), device=device)

    def step(self):
        return torch._scaled_mm(self.x, self.w.t(), scale_a=self.sx, scale_b=self.sw, out_dtype=torch.bfloat16)
