"""MoE token dispatch / combine over peer memory (see ``csrc/kernels/moe_dispatch.cu``).

``MoeAllToAll`` owns, per rank, a receive arena (``world`` regions of
``capacity`` rows), the 16-byte row headers and the flag block, all
peer-mapped. ``dispatch`` routes and pushes rows to the expert ranks,
``expert_ready`` is where an expert GEMM would run (identity here) and
``combine`` pulls the rows back with the gate-weighted sum fused into the read.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch

from . import _native
from ..parallel.peer import PeerGroup, SymmetricBuffer

_launches = 0


def launch_count() -> int:
    return _launches


def row_bytes(hidden: int, fp8: bool) -> int:
    """Bytes of one row in a receive arena (the kernels' layout: ``eux_moe_row_bytes``)."""
    return int(_native.load().eux_moe_row_bytes(hidden, 1 if fp8 else 0))


class MoeAllToAll:
    def __init__(self, group: PeerGroup, n_tokens: int, hidden: int, topk: int, n_experts: int,
                 fp8: bool = False, capacity: Optional[int] = None,
                 buffers: Optional[tuple] = None, rank: Optional[int] = None):
        if n_experts % group.world or hidden % 128:
            raise ValueError("n_experts must divide by world and hidden by 128")
        self.group = group
        self.rank = group.rank if rank is None else rank
        self.world = group.world
        self.n_tokens, self.hidden, self.topk, self.n_experts, self.fp8 = n_tokens, hidden, topk, n_experts, fp8
        self.capacity = capacity or n_tokens * topk
        self.row_bytes = row_bytes(hidden, fp8)
        epr = n_experts // self.world
        if buffers is None:
            arena = group.alloc(self.world * self.capacity * self.row_bytes)
            meta = group.alloc(self.world * self.capacity * 16)
            flags = group.alloc((3 * self.world + self.world * epr) * 8)
            buffers = (arena, meta, flags)
        self.arena, self.meta, self.flags = buffers
        dev = group.device
        self.slot_of = torch.empty(n_tokens * topk, dtype=torch.int32, device=dev)
        self.counters = torch.zeros(self.world + n_experts + 8, dtype=torch.int32, device=dev)
        self.status = torch.zeros(1, dtype=torch.int32, device=dev)
        self.out = torch.empty(n_tokens, hidden, dtype=torch.bfloat16, device=dev)
        self.seq = 0
        self._x = self._idx = self._w = None

    def close(self) -> None:
        """Collective release of the peer-mapped buffers: every rank calls it."""
        self.group.free(self.arena, self.meta, self.flags)

    @classmethod
    def emulated(cls, world: int, n_tokens: int, hidden: int, topk: int, n_experts: int, fp8: bool = False,
                 capacity: Optional[int] = None) -> List["MoeAllToAll"]:
        """``world`` logical ranks on one GPU (for single-device checks)."""
        g = PeerGroup.emulated(world)
        cap = capacity or n_tokens * topk
        rb = row_bytes(hidden, fp8)
        epr = n_experts // world
        arenas = g.alloc_emulated(world * cap * rb)
        metas = g.alloc_emulated(world * cap * 16)
        flags = g.alloc_emulated((3 * world + world * epr) * 8)
        return [cls(g, n_tokens, hidden, topk, n_experts, fp8, cap, (arenas[r], metas[r], flags[r]), rank=r)
                for r in range(world)]

    def _desc(self) -> _native.MoeDesc:
        d = _native.MoeDesc()
        d.rank, d.world, d.n_tokens, d.hidden = self.rank, self.world, self.n_tokens, self.hidden
        d.topk, d.n_experts, d.fp8, d.capacity = self.topk, self.n_experts, int(self.fp8), self.capacity
        d.x = self._x.data_ptr() if self._x is not None else None
        d.topk_idx = self._idx.data_ptr() if self._idx is not None else None
        d.topk_w = self._w.data_ptr() if self._w is not None else None
        d.arena_peer = self.arena.ptr_table.data_ptr()
        d.meta_peer = self.meta.ptr_table.data_ptr()
        d.flag_peer = self.flags.ptr_table.data_ptr()
        d.slot_of, d.counters, d.out = self.slot_of.data_ptr(), self.counters.data_ptr(), self.out.data_ptr()
        d.seq, d.wait_timeout_ns, d.status = self.seq, 2_000_000_000, self.status.data_ptr()
        return d

    def dispatch(self, x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, ctas: int = 0) -> None:
        global _launches
        assert x.dtype == torch.bfloat16 and x.is_contiguous() and x.shape == (self.n_tokens, self.hidden)
        assert topk_idx.dtype == torch.int32 and topk_w.dtype == torch.float32
        self._x, self._idx, self._w = x, topk_idx.contiguous(), topk_w.contiguous()
        self.seq += 1
        d = self._desc()
        _native.check(_native.load().eux_moe_dispatch_launch(C.byref(d), ctas, C.c_void_p(_native.current_stream_ptr())),
                      "eux_moe_dispatch_launch")
        _launches += 2

    def expert_ready(self) -> None:
        global _launches
        d = self._desc()
        _native.check(_native.load().eux_moe_expert_ready_launch(C.byref(d), C.c_void_p(_native.current_stream_ptr())),
                      "eux_moe_expert_ready_launch")
        _launches += 1

    def combine(self, ctas: int = 0) -> torch.Tensor:
        global _launches
        d = self._desc()
        _native.check(_native.load().eux_moe_combine_launch(C.byref(d), ctas, C.c_void_p(_native.current_stream_ptr())),
                      "eux_moe_combine_launch")
        _launches += 1
        return self.out

    # -- views for tests / expert code --------------------------------------
    def recv_counts(self) -> torch.Tensor:
        """rows received from each source rank (valid after expert_ready)."""
        epr = self.n_experts // self.world
        return self.flags.view(torch.int64, 3 * self.world + self.world * epr)[self.world:2 * self.world]

    def recv_rows(self, src: int, n: int) -> torch.Tensor:
        off = src * self.capacity * self.row_bytes
        return self.arena.local[off: off + n * self.row_bytes].view(n, self.row_bytes)

    def recv_meta(self, src: int, n: int) -> torch.Tensor:
        off = src * self.capacity * 16
        return self.meta.local[off: off + n * 16].view(torch.int32).view(n, 4)

    def check_status(self) -> None:
        s = int(self.status.item())
        if s:
            raise RuntimeError(f"moe kernel status code={s & 0xff} where={s >> 8}")


def reference_dispatch_combine(x: torch.Tensor, topk_idx: torch.Tensor, topk_w: torch.Tensor, fp8: bool) -> torch.Tensor:
    """Plain PyTorch fp32 statement of dispatch -> identity expert -> weighted combine."""
    xf = x.float()
    if fp8:
        t, h = xf.shape
        g = xf.view(t, h // 128, 128)
        scale = g.abs().amax(-1, keepdim=True).clamp_min(1e-10) * (1.0 / 448.0)
        q = (g * (1.0 / scale)).to(torch.float8_e4m3fn).float()
        xf = (q * scale).view(t, h)
    valid = (topk_idx >= 0).float()
    wsum = (topk_w * valid).sum(-1, keepdim=True)
    return xf * wsum
