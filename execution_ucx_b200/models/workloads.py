"""The named benchmark workloads as reusable classes over the data-plane ops.

Each class owns its peer-mapped buffers for one rank and exposes ``step()``
(one iteration, launched on the current stream) so that the bench, the tests
and user code drive exactly the same path.

Pairing: rank r talks to rank r^1 (with one rank, to itself: a loopback through
the same kernels and the same arena layout).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch

from ..ops import moe as moe_ops
from ..ops import remote_gemm as gemm_ops
from ..ops import tensor_xfer as tx
from ..parallel.peer import PeerGroup


def _partner(rank: int, world: int) -> int:
    return rank ^ 1 if world > 1 else rank


class TensorRpcEcho:
    """Axon tensor RPC, data plane only: the client pushes a tensor into the
    server's receive arena and publishes a sequence flag; the server's handler
    kernel (waiting on that flag, bounded) applies the handler and pushes the
    result straight back into the client's arena; the client's completion kernel
    waits for the echo flag. Every rank is client and server for its partner."""

    def __init__(self, group: PeerGroup, max_bytes: int, dtype=torch.bfloat16, handler_op: int = tx.OP_NONE,
                 handler_arg: float = 0.0):
        self.g, self.dtype = group, dtype
        self.peer = _partner(group.rank, group.world)
        self.max_bytes = max_bytes
        # arena layout per rank: [request slot | response slot]
        self.arena = group.alloc(2 * max_bytes)
        self.flags = group.alloc(256)          # [0]=request arrived, [1]=response arrived
        self.status = torch.zeros(1, dtype=torch.int32, device=group.device)
        self.handler_op, self.handler_arg = handler_op, handler_arg
        self.seq = 0
        self.esz = torch.empty((), dtype=dtype).element_size()

    def request_view(self, nbytes: int) -> torch.Tensor:
        return self.arena.view(self.dtype, nbytes // self.esz, 0)

    def response_view(self, nbytes: int) -> torch.Tensor:
        return self.arena.view(self.dtype, nbytes // self.esz, self.max_bytes)

    def step(self, src: torch.Tensor) -> torch.Tensor:
        """One echo round trip of ``src`` (device tensor); returns the response view."""
        nbytes = src.numel() * src.element_size()
        assert nbytes <= self.max_bytes
        self.seq += 1
        p = self.peer
        # client: push request into the partner's request slot
        tx.push(src, self.arena.peer_ptrs[p], dst_dtype=self.dtype, flag_ptr=self.flags.peer_ptrs[p], flag_value=self.seq)
        # server: wait for the partner's request, run the handler, push the response back
        req = self.request_view(nbytes)
        tx.push(req, self.arena.peer_ptrs[p] + self.max_bytes, dst_dtype=self.dtype, op=self.handler_op,
                op_arg=self.handler_arg, flag_ptr=self.flags.peer_ptrs[p] + 8, flag_value=self.seq,
                wait_flag_ptr=self.flags.local_ptr, wait_value=self.seq, status_ptr=self.status.data_ptr())
        # client: completion = the response flag (observed by a tiny wait kernel writing nothing)
        resp = self.response_view(nbytes)
        tx.push(resp[:8], self._sink(), wait_flag_ptr=self.flags.local_ptr + 8, wait_value=self.seq,
                status_ptr=self.status.data_ptr())
        return resp

    def _sink(self) -> torch.Tensor:
        if not hasattr(self, "_sink_t"):
            self._sink_t = torch.empty(8, dtype=self.dtype, device=self.g.device)
        return self._sink_t

    def check_status(self):
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"tensor rpc status code={s & 0xff} where={s >> 8}")


class DevicePingPong:
    """Latency/bandwidth of the data plane alone: one kernel per GPU runs the
    whole ping-pong on the device (no launches inside the timed loop)."""

    def __init__(self, group: PeerGroup, max_bytes: int):
        self.g = group
        self.peer = _partner(group.rank, group.world)
        self.buf = group.alloc(max_bytes)
        self.scratch = group.alloc(max_bytes) if group.world == 1 else None
        self.flags = group.alloc(256)
        dev = group.device
        self.bar = torch.zeros(2, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.seq = 0

    def run(self, nbytes: int, iters: int) -> torch.Tensor:
        """Returns per-iteration round-trip times in ns (device globaltimer), on the initiating rank."""
        ts = torch.zeros(iters + 1, dtype=torch.int64, device=self.g.device)
        if self.g.world == 1:
            tx.pingpong(self.buf.local, self.scratch.local_ptr, nbytes, 0, 0, self.bar, iters, 2, ts_out=ts,
                        status=self.status)
        else:
            init = 1 if self.g.rank < self.peer else 0
            tx.pingpong(self.buf.local, self.buf.peer_ptrs[self.peer], nbytes, self.flags.local_ptr,
                        self.flags.peer_ptrs[self.peer], self.bar, iters, init, base_seq=self.seq, ts_out=ts,
                        status=self.status)
            self.seq += iters
        torch.cuda.synchronize()
        if int(self.status.item()):
            raise RuntimeError("ping-pong wait ran out")
        return ts[1:] - ts[:-1]


class RemoteGemmRpc:
    """Remote-GEMM RPC: this rank is callee for its partner's X and caller of
    its partner's weight. X lives in the caller's arena; the callee kernel pulls
    it panel by panel while computing and stores Y into the caller's arena."""

    def __init__(self, group: PeerGroup, m: int, n: int, k: int, copy_ctas: int = 12):
        self.g, self.m, self.n, self.k, self.copy_ctas = group, m, n, k, copy_ctas
        self.peer = _partner(group.rank, group.world)
        dev = group.device
        self.x_buf = group.alloc(m * k * 2)
        self.y_buf = group.alloc(m * n * 2)
        self.flags = group.alloc(256)
        self.x = self.x_buf.view(torch.bfloat16, m * k).view(m, k)
        self.y = self.y_buf.view(torch.bfloat16, m * n).view(m, n)
        g = torch.Generator(device=dev).manual_seed(1234 + group.rank)
        self.x.copy_(torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16))
        self.w = (torch.randn(k, n, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        self.gemm = gemm_ops.RemoteGemm(self.w, m)
        self.seq = 0
        self.sink = torch.empty(8, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        group.barrier()

    def step(self) -> torch.Tensor:
        self.seq += 1
        p = self.peer
        local = self.g.world == 1
        # callee: consume the partner's X from its memory, write Y into the partner's memory
        self.gemm(self.x_buf.peer_ptrs[p], self.m, self.y_buf.peer_ptrs[p], x_is_local=False,
                  done_flag_ptr=self.flags.peer_ptrs[p], done_value=self.seq, copy_ctas=self.copy_ctas)
        # caller: wait until the partner has delivered Y here
        tx.push(self.y.view(-1)[:8], self.sink, wait_flag_ptr=self.flags.local_ptr, wait_value=self.seq,
                status_ptr=self.status.data_ptr())
        return self.y

    def check(self):
        self.gemm.check_status()
        if int(self.status.item()):
            raise RuntimeError("remote gemm completion wait ran out")


class MoeDispatchCombine:
    """MoE token dispatch -> identity expert -> gate-weighted combine on all ranks."""

    def __init__(self, group: PeerGroup, n_tokens: int = 4096, hidden: int = 7168, topk: int = 8,
                 n_experts: int = 256, fp8: bool = False, seed: int = 0):
        self.g = group
        dev = group.device
        self.a2a = moe_ops.MoeAllToAll(group, n_tokens, hidden, topk, n_experts, fp8=fp8)
        g = torch.Generator(device=dev).manual_seed(seed + 17 * group.rank)
        self.x = torch.randn(n_tokens, hidden, device=dev, generator=g).to(torch.bfloat16)
        scores = torch.rand(n_tokens, n_experts, device=dev, generator=g)
        self.idx = scores.topk(topk, dim=-1).indices.to(torch.int32)
        self.w = torch.softmax(torch.randn(n_tokens, topk, device=dev, generator=g), dim=-1)
        self.fp8 = fp8
        group.barrier()

    def step(self) -> torch.Tensor:
        self.a2a.dispatch(self.x, self.idx, self.w)
        self.a2a.expert_ready()
        return self.a2a.combine()

    def reference(self) -> torch.Tensor:
        return moe_ops.reference_dispatch_combine(self.x, self.idx, self.w, self.fp8)

    def bytes_per_direction(self) -> int:
        return self.a2a.n_tokens * self.a2a.topk * self.a2a.row_bytes
