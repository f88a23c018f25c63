"""Symmetric device buffers whose handles travel through the runtime's own control plane.

``AxonPeerMemory`` gives the same ``SymmetricBuffer`` objects as ``PeerGroup.alloc`` (a local
region plus a table of every rank's region as seen from this GPU), but nothing here touches
``torch.distributed``: every rank allocates from its runtime's CUDA memory resource, exports
the region and announces it to its peers with an Axon call (an active message over the
runtime's context); the peers map it with ``import_region``. The kernels of the all-to-all
workloads are then launched on those tables.
"""
from __future__ import annotations

import asyncio
from typing import List

import torch

from .peer import SymmetricBuffer


class _DeviceView:
    """Lets torch view runtime-owned device memory (no ownership: the runtime frees it)."""

    def __init__(self, ptr: int, nbytes: int):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (ptr, False), "version": 3, "strides": None}


class AxonPeerMemory:
    def __init__(self, runtime, rank: int, world: int, worker_names: List[str], device: torch.device):
        """``worker_names[r]`` is the name under which rank r's runtime is connected (unused at ``rank``)."""
        self.rt, self.rank, self.world, self.names, self.device = runtime, rank, world, list(worker_names), device
        runtime.peer_memory_init(rank, world)
        self._next_tag = 1
        self._tags = {}

    async def alloc(self, nbytes: int, timeout_s: float = 30.0) -> SymmetricBuffer:
        """Collective: every rank calls it with the same size, in the same order."""
        nbytes = (nbytes + 255) // 256 * 256
        tag = self._next_tag
        self._next_tag += 1
        ptr = self.rt.peer_memory_alloc(tag, nbytes)
        others = [n for r, n in enumerate(self.names) if r != self.rank]
        if others:
            await asyncio.gather(*[self.rt.peer_memory_publish(n, tag) for n in others])
            waited = 0.0
            while self.rt.peer_memory_arrived(tag) < self.world - 1:
                await asyncio.sleep(0.0005)
                waited += 0.0005
                if waited > timeout_s:
                    raise TimeoutError(f"peer memory: only {self.rt.peer_memory_arrived(tag)} of {self.world - 1} peers announced buffer {tag}")
        ptrs = list(self.rt.peer_memory_resolve(tag))
        local = torch.as_tensor(_DeviceView(ptr, nbytes), device=self.device)
        table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        buf = SymmetricBuffer(nbytes, self.rank, ptrs, local, table, [], [])
        self._tags[id(buf)] = tag
        return buf

    def free(self, *bufs: SymmetricBuffer) -> None:
        """Gives this rank's regions back. The caller makes sure (a barrier of its own) that no peer's kernel
        still reads or writes them."""
        for b in bufs:
            tag = self._tags.pop(id(b), None) if b is not None else None
            if tag is not None:
                self.rt.peer_memory_free(tag)
