"""Peer-mapped ("symmetric") device buffers for the data-plane kernels.

One process per GPU. Each rank allocates a buffer with ``cudaMalloc``, exports
it with a CUDA IPC handle, exchanges the 64-byte handles over the control plane
(any ``torch.distributed`` backend: NCCL on GPUs, gloo in CPU tests) and maps
every peer's buffer. Kernels then receive a device table ``ptrs[world]`` and
store straight into the destination GPU's memory over NVLink.

This mirrors, for the Python benches, what the C++ ``CudaMemoryResourceManager``
does for the runtime (register + export + peer-map), in the place where the
reference registers memory with ``ucp_mem_map``
(ucx_context/ucx_am_context/ucx_am_context.cpp:1128-1147).

``PeerGroup.emulated(world)`` builds the same tables for ``world`` logical ranks
that all live on one GPU: the multi-rank kernels can then be checked on a single
device, one logical rank per launch, launches in sequence on one stream.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field
from typing import List, Optional

import torch

from ..ops import _native


class _RawCudaBuffer:
    """Owner of one cudaMalloc allocation, viewable as a torch tensor."""

    def __init__(self, nbytes: int, free_on_del: bool = True):
        # free_on_del is off for memory that other processes map: its release is collective
        self.free_on_del = free_on_del
        lib = _native.load()
        p = C.c_void_p()
        _native.check(lib.eux_device_malloc(C.byref(p), nbytes), "cudaMalloc")
        self.ptr = p.value
        self.nbytes = nbytes
        self.__cuda_array_interface__ = {
            "shape": (nbytes,), "typestr": "|u1", "data": (self.ptr, False), "version": 3, "strides": None,
        }

    def free(self):
        if self.ptr:
            _native.load().eux_device_free(C.c_void_p(self.ptr))
            self.ptr = 0

    def __del__(self):
        try:
            if self.free_on_del:
                self.free()
        except Exception:
            pass


@dataclass
class SymmetricBuffer:
    """A buffer that exists once per rank; ``peer_ptrs[r]`` is rank r's copy as
    seen from this process (``peer_ptrs[rank]`` is the local one)."""
    nbytes: int
    rank: int
    peer_ptrs: List[int]
    local: torch.Tensor                      # uint8 view of the local copy
    ptr_table: torch.Tensor                  # int64[world] on the device
    _owners: list = field(default_factory=list, repr=False)
    _opened: list = field(default_factory=list, repr=False)

    @property
    def local_ptr(self) -> int:
        return self.peer_ptrs[self.rank]

    def view(self, dtype, numel: int, byte_offset: int = 0) -> torch.Tensor:
        esz = torch.empty((), dtype=dtype).element_size()
        return self.local[byte_offset:byte_offset + numel * esz].view(dtype)

    def unmap_peers(self):
        lib = _native.load()
        for p in self._opened:
            lib.eux_ipc_close(C.c_void_p(p))
        self._opened.clear()

    def free_local(self):
        for o in self._owners:
            o.free()
        self._owners.clear()

    def close(self):
        """Single-process teardown. With several ranks use ``PeerGroup.free``: a rank must not free
        its copy while a peer still has it mapped (the next allocation could get the same memory,
        and the peer could not map it a second time)."""
        self.unmap_peers()
        self.free_local()


class PeerGroup:
    """The set of ranks that can reach each other's memory."""

    def __init__(self, rank: int = 0, world: int = 1, device: Optional[torch.device] = None,
                 dist_group=None, emulated: bool = False):
        self.rank, self.world, self.emulated_mode = rank, world, emulated
        self.device = device or torch.device("cuda", torch.cuda.current_device())
        self.dist_group = dist_group

    @classmethod
    def from_env(cls) -> "PeerGroup":
        """Build from torch.distributed (already initialised) or a single process."""
        import torch.distributed as dist
        if dist.is_available() and dist.is_initialized():
            return cls(dist.get_rank(), dist.get_world_size())
        return cls(0, 1)

    @classmethod
    def emulated(cls, world: int) -> "PeerGroup":
        return cls(0, world, emulated=True)

    # -- allocation ---------------------------------------------------------
    def free(self, *bufs: "SymmetricBuffer") -> None:
        """Collective release: every rank drops its mappings of the peers' copies, then (after a
        barrier) frees its own copy. Memory is not given back when a buffer is merely dropped."""
        torch.cuda.synchronize()
        self.barrier()
        for b in bufs:
            if b is not None:
                b.unmap_peers()
        self.barrier()
        for b in bufs:
            if b is not None:
                b.free_local()
        self.barrier()

    def alloc(self, nbytes: int) -> SymmetricBuffer:
        # whole 2 MiB blocks: an allocation then never shares its exported block with another one
        nbytes = (nbytes + (2 << 20) - 1) // (2 << 20) * (2 << 20)
        if self.emulated_mode:
            raise RuntimeError("use alloc_emulated() on an emulated group")
        lib = _native.load()
        own = _RawCudaBuffer(nbytes, free_on_del=self.world == 1)
        local = torch.as_tensor(own, device=self.device)
        local.zero_()
        torch.cuda.synchronize()
        ptrs = [0] * self.world
        ptrs[self.rank] = own.ptr
        opened = []
        if self.world > 1:
            import torch.distributed as dist
            handle = C.create_string_buffer(64)
            _native.check(lib.eux_ipc_export(C.c_void_p(own.ptr), handle), "cudaIpcGetMemHandle")
            gathered = [None] * self.world
            dist.all_gather_object(gathered, bytes(handle.raw), group=self.dist_group)
            for r, h in enumerate(gathered):
                if r == self.rank:
                    continue
                p = C.c_void_p()
                _native.check(lib.eux_ipc_open(C.c_char_p(h), C.byref(p)), f"cudaIpcOpenMemHandle(rank {r})")
                ptrs[r] = p.value
                opened.append(p.value)
            dist.barrier(group=self.dist_group)
        table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        return SymmetricBuffer(nbytes, self.rank, ptrs, local, table, [own], opened)

    def alloc_emulated(self, nbytes: int) -> List[SymmetricBuffer]:
        """``world`` local buffers wired up as if each belonged to another rank."""
        nbytes = (nbytes + 255) // 256 * 256
        owners = [_RawCudaBuffer(nbytes) for _ in range(self.world)]
        ptrs = [o.ptr for o in owners]
        table = torch.tensor(ptrs, dtype=torch.int64, device=self.device)
        out = []
        for r in range(self.world):
            local = torch.as_tensor(owners[r], device=self.device)
            local.zero_()
            out.append(SymmetricBuffer(nbytes, r, list(ptrs), local, table, [owners[r]], []))
        torch.cuda.synchronize()
        return out

    def barrier(self):
        if self.world > 1 and not self.emulated_mode:
            import torch.distributed as dist
            dist.barrier(group=self.dist_group)

    def max_over_ranks(self, value: float) -> float:
        """Max of a host scalar over ranks (used for device-timed durations)."""
        if self.world > 1 and not self.emulated_mode:
            import torch.distributed as dist
            t = torch.tensor([value], dtype=torch.float64, device=self.device)
            dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.dist_group)
            return float(t.item())
        return value
