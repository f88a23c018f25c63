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
    waits for the echo flag. Every rank is client and server for its partner.
    With ``fused`` (the default) the three roles of a step run as the phases of one kernel launch per
    rank; a strided or differently typed source takes the three launches."""

    def __init__(self, group: PeerGroup, max_bytes: int, dtype=torch.bfloat16, handler_op: int = tx.OP_NONE,
                 handler_arg: float = 0.0, fused: bool = True):
        self.g, self.dtype = group, dtype
        self.fused = fused   # one launch per step where the source allows it (dense, arena dtype, 16-byte aligned)
        self._steps = {}     # prepared descriptors per (source address, size)
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
        if self.fused and src.is_contiguous() and src.dtype == self.dtype and src.data_ptr() % 16 == 0:
            key = (src.data_ptr(), nbytes)
            hit = self._steps.get(key)
            if hit is None:
                if len(self._steps) >= 64:
                    self._steps.clear()
                hit = (tx.RpcEchoStep(src, self.arena.peer_ptrs[p], self.flags.peer_ptrs[p], self.request_view(nbytes),
                                      self.arena.peer_ptrs[p] + self.max_bytes, self.flags.peer_ptrs[p] + 8,
                                      self.flags.local_ptr, self.flags.local_ptr + 8, op=self.handler_op,
                                      op_arg=self.handler_arg, status_ptr=self.status.data_ptr()),
                       self.response_view(nbytes))
                self._steps[key] = hit
            hit[0].launch(self.seq)
            return hit[1]
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

    def close(self):
        """Collective: every rank calls it."""
        self.g.free(self.arena, self.flags)


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

    def close(self):
        """Collective: every rank calls it."""
        self.g.free(self.buf, self.scratch, self.flags)


class RemoteGemmRpc:
    """Remote-GEMM RPC: this rank is callee for its partner's X and caller of
    its partner's weight. X lives in the caller's arena; the callee kernel pulls
    it panel by panel while computing and stores Y into the caller's arena.
    With ``fp8`` the caller sends e4m3 rows with one fp32 scale per 128 elements
    and the resident weight is e4m3 with 128x128 block scales; with ``fp8="mx"``
    both operands are MXFP8 (a power-of-two scale per 32 elements, applied by the
    tensor core). A single rank has nothing to pull: its kernel reads X in place."""

    def __init__(self, group: PeerGroup, m: int, n: int, k: int, copy_ctas: int = 0, fp8: bool = False):
        self.g, self.m, self.n, self.k, self.copy_ctas, self.fp8 = group, m, n, k, copy_ctas, fp8
        self.peer = _partner(group.rank, group.world)
        dev = group.device
        self.x_buf = group.alloc(m * k * (1 if fp8 else 2))
        self.y_buf = group.alloc(m * n * 2)
        self.flags = group.alloc(256)
        self.y = self.y_buf.view(torch.bfloat16, m * n).view(m, n)
        g = torch.Generator(device=dev).manual_seed(1234 + group.rank)
        x = torch.randn(m, k, device=dev, generator=g).to(torch.bfloat16)
        self.w = (torch.randn(k, n, device=dev, generator=g) * 0.02).to(torch.bfloat16)
        if fp8 == "mx":
            xq, xsf = gemm_ops.quantize_mx(x)
            chunks = gemm_ops.mx_scale_chunks(xsf, False)
            self.xs_buf = group.alloc(chunks.numel())
            self.xq = self.x_buf.view(torch.uint8, m * k).view(m, k)
            self.xs = self.xs_buf.view(torch.uint8, chunks.numel())
            self.xq.copy_(xq.view(torch.uint8))
            self.xs.copy_(chunks)
            self.x_sf = xsf
            self.gemm = gemm_ops.RemoteGemmMx(self.w.float(), m)
            self.x = x
        elif fp8:
            xq, xs = gemm_ops.quantize_rows_1x128(x)
            self.xs_buf = group.alloc(m * (k // 128) * 4)
            self.xq = self.x_buf.view(torch.uint8, m * k).view(m, k)
            self.xs = self.xs_buf.view(torch.float32, m * (k // 128)).view(m, k // 128)
            self.xq.copy_(xq.view(torch.uint8))
            self.xs.copy_(xs)
            self.gemm = gemm_ops.RemoteGemmFp8(self.w, m)
            self.x = x
        else:
            self.x = self.x_buf.view(torch.bfloat16, m * k).view(m, k)
            self.x.copy_(x)
            self.gemm = gemm_ops.RemoteGemm(self.w, m)
        self.seq = 0
        self.sink = torch.empty(8, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        group.barrier()

    def step(self) -> torch.Tensor:
        self.seq += 1
        p = self.peer
        local = self.g.world == 1
        kw = dict(x_is_local=local, done_flag_ptr=self.flags.peer_ptrs[p], done_value=self.seq,
                  copy_ctas=0 if local else self.copy_ctas)
        # callee: consume the partner's X from its memory, write Y into the partner's memory
        if self.fp8:
            self.gemm(self.x_buf.peer_ptrs[p], self.xs_buf.peer_ptrs[p], self.m, self.y_buf.peer_ptrs[p], **kw)
        else:
            self.gemm(self.x_buf.peer_ptrs[p], self.m, self.y_buf.peer_ptrs[p], **kw)
        # caller: wait until the partner has delivered Y here
        tx.push(self.y.view(-1)[:8], self.sink, wait_flag_ptr=self.flags.local_ptr, wait_value=self.seq,
                status_ptr=self.status.data_ptr())
        return self.y

    def reference_rows(self, rows: int = 256) -> torch.Tensor:
        """fp32 reference of the first rows (single rank: X and W are both local)."""
        if self.fp8 == "mx":
            return gemm_ops.mx_dequantized_reference(self.xq[:rows].view(torch.float8_e4m3fn), self.x_sf[:rows],
                                                     self.gemm.w_q_t, self.gemm.w_sf)
        if self.fp8:
            return gemm_ops.dequantized_reference(self.xq[:rows].view(torch.float8_e4m3fn), self.xs[:rows],
                                                  self.gemm.w_q_t, self.gemm.w_scale)
        return self.x[:rows].float() @ self.w.float()

    def check(self):
        self.gemm.check_status()
        if int(self.status.item()):
            raise RuntimeError("remote gemm completion wait ran out")

    def close(self):
        """Collective: every rank calls it."""
        self.g.free(self.x_buf, self.y_buf, self.flags, getattr(self, "xs_buf", None))


class RemoteGemmAxon:
    """The remote-GEMM RPC through the runtime: every rank serves its weight with ``AxonRuntime.serve_gemm``
    and calls its partner's with ``AxonRuntime.remote_gemm``. The request is a small active message that
    describes the caller's X and Y regions (exported by the memory resource); the callee's handler maps them
    and launches the GEMM kernel on them; the reply is the kernel's status. ``peers="all"``: every rank calls
    every other rank's weight in one step (world - 1 calls in flight per rank)."""

    def __init__(self, api: "AxonTensorRpc", m: int, n: int, k: int, fmt: str = "bf16", peers: str = "partner",
                 weight_id: Optional[int] = None):
        self.api, self.m, self.n, self.k, self.fmt = api, m, n, k, fmt
        g = api.group
        dev = g.device
        gen = torch.Generator(device=dev).manual_seed(1234 + g.rank)
        x = torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16)
        self.w = (torch.randn(k, n, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.x_ref = x
        self.x_scale = None
        if fmt == "bf16":
            self.x = x
        elif fmt in ("fp8_block", "fp8_block_pow2"):
            # "fp8_block": arbitrary fp32 scales on both sides (served by the kernel that applies them in its
            # epilogue); "fp8_block_pow2": the same format with power-of-two scales (served by the MX kernel)
            self.x, self.x_scale = gemm_ops.quantize_rows_1x128(x, pow2=fmt == "fp8_block_pow2")
        else:
            self.x, sf = gemm_ops.quantize_mx(x)
            self.x_sf = sf
            self.x_scale = gemm_ops.mx_scale_chunks(sf, False)
        self.weight_id = weight_id if weight_id is not None else {"bf16": 1, "fp8_block": 2, "mxfp8": 3, "fp8_block_pow2": 4}[fmt]
        self.pow2 = fmt == "fp8_block_pow2"
        # the scales as they are sent: fp32 per 1x128 block, or (power-of-two route) their MX form, made once with X
        self.x_scale_sent = gemm_ops.mx_scale_chunks(gemm_ops.block_scales_to_mx(self.x_scale, 1), False) if self.pow2 else self.x_scale
        if self.pow2:
            api.server.serve_gemm(self.weight_id, self.w, "fp8_block", max_m=m, pow2_scales=True)
        else:
            api.server.serve_gemm(self.weight_id, self.w, fmt, max_m=m, pow2_scales=False)
        if g.world == 1:
            self.targets = [api.partner_name]
        elif peers == "all":
            self.targets = [f"axon{(g.rank + 1 + i) % g.world}" for i in range(g.world - 1)]
        else:
            self.targets = [api.partner_name]
        self.ys = [torch.zeros(m, n, dtype=torch.bfloat16, device=dev) for _ in self.targets]
        torch.cuda.synchronize()

    async def step(self):
        import asyncio
        futs = [self.api.client.remote_gemm(self.x, y, worker_name=t, weight_id=self.weight_id, x_scale=self.x_scale_sent, x_scale_pow2=self.pow2)
                for t, y in zip(self.targets, self.ys)]
        # one call: awaited as it is (gathering it would cost one more turn of the event loop)
        status = [await futs[0]] if len(futs) == 1 else await asyncio.gather(*futs)
        if any(status):
            raise RuntimeError(f"remote gemm kernel status {status}")
        return self.ys[0]

    def callee_seed_rank(self, target: str) -> int:
        return int(target[4:]) if target.startswith("axon") and target[4:].isdigit() else self.api.group.rank

    def reference_rows(self, target_index: int = 0, rows: int = 256) -> torch.Tensor:
        """fp32 reference of the first rows of the result of ``targets[target_index]``: the callee's weight is
        rebuilt here from its seed, so the check needs nothing from the callee but the result itself."""
        dev = self.api.group.device
        r = self.callee_seed_rank(self.targets[target_index])
        gen = torch.Generator(device=dev).manual_seed(1234 + r)
        torch.randn(self.m, self.k, device=dev, generator=gen)                 # the callee's own X comes first in its stream
        w = (torch.randn(self.k, self.n, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        if self.fmt == "bf16":
            return self.x_ref[:rows].float() @ w.float()
        if self.fmt in ("fp8_block", "fp8_block_pow2"):
            wq, ws = gemm_ops.quantize_blocks_128x128(w.t().contiguous(), pow2=self.pow2)
            return gemm_ops.dequantized_reference(self.x[:rows], self.x_scale[:rows], wq, ws)
        wq, wsf = gemm_ops.quantize_mx(w.float().t().contiguous())
        return gemm_ops.mx_dequantized_reference(self.x[:rows], self.x_sf[:rows], wq, wsf)

    def max_abs_err(self, rows: int = 256) -> float:
        return max(float((y[:rows].float() - self.reference_rows(i, rows)).abs().max()) for i, y in enumerate(self.ys))


class RemoteGemmAllPeers:
    """Every rank calls the remote GEMM of every other rank: as callee a rank runs one fused
    kernel per caller (pulling that caller's X, storing Y into the caller's slot for this callee),
    as caller it waits for the world-1 results. Callers are served in a rotated order so that no
    rank's X is pulled by everybody at once."""

    def __init__(self, group: PeerGroup, m: int, n: int, k: int):
        self.g, self.m, self.n, self.k = group, m, n, k
        dev, w = group.device, group.world
        self.x_buf = group.alloc(m * k * 2)
        self.y_slot = m * n * 2
        self.y_buf = group.alloc(self.y_slot * w)
        self.flags = group.alloc(8 * w)
        gen = torch.Generator(device=dev).manual_seed(77 + group.rank)
        self.x = self.x_buf.view(torch.bfloat16, m * k).view(m, k)
        self.x.copy_(torch.randn(m, k, device=dev, generator=gen).to(torch.bfloat16))
        self.w = (torch.randn(k, n, device=dev, generator=gen) * 0.02).to(torch.bfloat16)
        self.gemm = gemm_ops.RemoteGemm(self.w, m)
        self.order = [(group.rank + 1 + i) % w for i in range(w - 1)]
        self.seq = 0
        self.sink = torch.empty(8, dtype=torch.bfloat16, device=dev)
        self.probe = torch.zeros(8, dtype=torch.bfloat16, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        group.barrier()

    def step(self) -> None:
        self.seq += 1
        r = self.g.rank
        for p in self.order:      # callee for caller p
            self.gemm(self.x_buf.peer_ptrs[p], self.m, self.y_buf.peer_ptrs[p] + r * self.y_slot, x_is_local=False,
                      done_flag_ptr=self.flags.peer_ptrs[p] + 8 * r, done_value=self.seq)
        for p in self.order:      # caller: the result of callee p has landed in slot p
            tx.push(self.probe, self.sink, wait_flag_ptr=self.flags.local_ptr + 8 * p, wait_value=self.seq,
                    status_ptr=self.status.data_ptr())

    def check(self):
        self.gemm.check_status()
        if int(self.status.item()):
            raise RuntimeError("a remote gemm result did not arrive in time")

    def close(self):
        """Collective: every rank calls it."""
        self.g.free(self.x_buf, self.y_buf, self.flags)


class MoeAxon:
    """MoE dispatch -> expert -> gate-weighted combine whose arenas, row headers and flag blocks come from the
    runtime's CUDA memory resource and whose handles were exchanged by Axon calls (``AxonPeerMemory``), not by
    ``torch.distributed``. The kernels are the same as ``MoeDispatchCombine``'s. ``expert_scale``: the expert is
    not the identity but multiplies what it received for local expert e by ``1 + e / 256``, so that a combine
    which paired a row with the wrong weight or the wrong expert's copy cannot pass for correct."""

    @classmethod
    async def create(cls, api: "AxonTensorRpc", n_tokens: int = 4096, hidden: int = 7168, topk: int = 8, n_experts: int = 256,
                     fp8: bool = False, seed: int = 0) -> "MoeAxon":
        from ..parallel.axon_peer import AxonPeerMemory
        self = cls()
        g = api.group
        self.api, self.g, self.fp8 = api, g, fp8
        rt = api.server
        if getattr(api, "peer_memory", None) is None:
            api.peer_memory = AxonPeerMemory(rt, g.rank, g.world, api.names, g.device)
            await api.barrier()        # every rank serves the announcement function before anybody announces
        pm = self.pm = api.peer_memory
        rb = moe_ops.row_bytes(hidden, fp8)
        cap = n_tokens * topk
        epr = n_experts // g.world
        arena = await pm.alloc(g.world * cap * rb)
        meta = await pm.alloc(g.world * cap * 16)
        flags = await pm.alloc((3 * g.world + g.world * epr) * 8)
        self.bufs = (arena, meta, flags)
        self.a2a = moe_ops.MoeAllToAll(g, n_tokens, hidden, topk, n_experts, fp8=fp8, capacity=cap, buffers=self.bufs)
        dev = g.device
        gen = torch.Generator(device=dev).manual_seed(seed + 17 * g.rank)
        self.x = torch.randn(n_tokens, hidden, device=dev, generator=gen).to(torch.bfloat16)
        scores = torch.rand(n_tokens, n_experts, device=dev, generator=gen)
        self.idx = scores.topk(topk, dim=-1).indices.to(torch.int32)
        self.w = torch.softmax(torch.randn(n_tokens, topk, device=dev, generator=gen), dim=-1)
        torch.cuda.synchronize()
        await api.barrier()
        return self

    def step(self) -> torch.Tensor:
        self.a2a.dispatch(self.x, self.idx, self.w)
        self.a2a.expert_ready()
        return self.a2a.combine()

    def reference(self) -> torch.Tensor:
        return moe_ops.reference_dispatch_combine(self.x, self.idx, self.w, self.fp8)

    def bytes_per_direction(self) -> int:
        return self.a2a.n_tokens * self.a2a.topk * self.a2a.row_bytes

    async def close(self):
        torch.cuda.synchronize()
        await self.api.barrier()
        self.pm.free(*self.bufs)
        await self.api.barrier()


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


class AxonTensorRpc:
    """Tensor echo through the public RPC API: ``AxonRuntime.register_function`` on the serving
    side, ``AxonRuntime.invoke`` on the calling side, device tensors both ways.

    With one rank the server and the client runtime live in this process on the same GPU; with more,
    every rank runs one runtime that serves ``echo`` and calls it on its partner (rank r with r^1).
    Request and response land in buffers that the memory policies hand out, allocated once per shape,
    so the steady state allocates nothing. The control messages travel through the runtime's shared-memory
    rings; the tensor bytes are moved by its transfer kernels over the peer mapping: stored into the
    receiver's ring up to the eager limit (no policy is asked then), pushed into the policy's buffer above it.
    """

    def __init__(self, group: PeerGroup, dtype=torch.bfloat16, timeout_ms: int = 60000):
        from .. import axon
        self.axon, self.group, self.dtype = axon, group, dtype
        self.g = group
        self.dev = group.device
        self.rank, self.world = group.rank, group.world
        self._srv_bufs, self._cli_bufs = {}, {}
        self.server = self.client = None
        self.partner_name = None
        self.timeout_ms = timeout_ms

    def _policy(self, cache):
        def policy(metas):
            key = tuple(metas[0].shape)
            buf = cache.get(key)
            if buf is None:
                buf = cache[key] = torch.empty(key, dtype=self.dtype, device=self.dev)
            return buf
        return policy

    async def start(self, connect_all: bool = False):
        """``connect_all``: connect to every rank's runtime, not only to the partner's (the all-to-all workloads)."""
        axon = self.axon
        index = self.dev.index or 0
        device = (lambda i: axon.cuda(i)) if self.dev.type == "cuda" else (lambda i: None)

        async def echo(x: torch.Tensor) -> torch.Tensor:
            return x

        if self.world == 1:
            self.server = axon.AxonRuntime("axon_srv", timeout=self.timeout_ms, device=device(index))
            self.client = axon.AxonRuntime("axon_cli", timeout=self.timeout_ms, device=device(index))
            self.server.register_function(echo, memory_policy=self._policy(self._srv_bufs))
            self.server.start_server()
            self.client.start_client()
            self.partner_name = "axon_srv"
            self.names = ["axon_srv"]
            await self.client.connect_endpoint_async(self.server.get_local_address(), self.partner_name)
            return
        import torch.distributed as dist
        me = f"axon{self.rank}"
        rt = axon.AxonRuntime(me, timeout=self.timeout_ms, device=device(index))
        rt.register_function(echo, memory_policy=self._policy(self._srv_bufs))
        rt.start()
        self.server = self.client = rt
        addrs = [None] * self.world
        dist.all_gather_object(addrs, bytes(rt.get_local_address()))
        partner = _partner(self.rank, self.world)
        self.partner_name = f"axon{partner}"
        self.names = [f"axon{r}" for r in range(self.world)]
        await rt.connect_endpoint_async(addrs[partner], self.partner_name)
        if connect_all:
            for r in range(self.world):
                if r not in (self.rank, partner):
                    await rt.connect_endpoint_async(addrs[r], self.names[r])
        await self.barrier()

    async def barrier(self):
        """A barrier that keeps this rank's event loop (and so its ``echo`` handler) running."""
        import asyncio
        if self.world == 1:
            return
        import torch.distributed as dist
        work = dist.barrier(async_op=True)
        while not work.is_completed():
            await asyncio.sleep(0.0005)

    async def step(self, x: torch.Tensor) -> torch.Tensor:
        return await self.client.invoke(x, worker_name=self.partner_name, session_id=1, function="echo",
                                        memory_policy=self._policy(self._cli_bufs))

    def transport_stats(self) -> dict:
        """Counters of this rank's runtime(s), added up."""
        out = dict(self.client.transport_stats())
        if self.server is not self.client:
            for k, v in self.server.transport_stats().items():
                out[k] = out.get(k, 0) + v
        return out

    def kernel_launches(self) -> int:
        """Transfer-kernel launches made so far by this rank's runtime(s)."""
        return int(self.transport_stats()["kernel_launches"])

    def stop(self):
        if self.client is not None:
            self.client.stop()
        if self.server is not None and self.server is not self.client:
            self.server.stop()
