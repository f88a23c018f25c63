"""Device descriptions handed to ``AxonRuntime(device=...)``.

The public surface is the one of the reference's ``axon/python/axon/device.py:12-299``:
a ``Device`` base with ``get_type()``, ``get_type_string()`` and ``get_context_handle()``,
the four concrete kinds with their keyword arguments (``CpuDevice(numa_node=)``,
``CudaDevice(device_id=, context=)``, ``RocmDevice(device_id=, context=)``,
``SyclDevice(device_id=, context=, queue=)``), the factory functions and ``auto_detect()``.

What differs underneath: this runtime binds a worker thread to a CUDA device by ordinal
(``cudaSetDevice``), not by pushing a driver context, so the "context handle" of a
``CudaDevice`` is informational: it is whatever the caller passed, or the ordinal of the
device that is current on the calling thread when a CUDA runtime is present. ``rocm`` and
``sycl`` devices can be described (code written for the reference imports and runs up to
that point) but a runtime cannot be started on them.

``kind`` / ``index`` are the two fields the native binding reads.
"""
from __future__ import annotations

import enum
from typing import Optional


class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    ROCM = "rocm"
    SYCL = "sycl"


class Device:
    """Base of the device descriptions. Subclasses set ``_type``."""

    _type: DeviceType = DeviceType.CPU

    def get_type(self) -> DeviceType:
        return self._type

    def get_type_string(self) -> str:
        return self._type.value

    def get_context_handle(self) -> Optional[int]:
        return None

    # ---- what the native runtime reads -------------------------------------------------
    @property
    def kind(self) -> str:
        return self._type.value

    @property
    def index(self) -> int:
        return int(getattr(self, "device_id", 0) or 0)

    @property
    def device_type(self) -> DeviceType:
        return self._type

    def is_available(self) -> bool:
        return False

    def __eq__(self, other) -> bool:
        return type(self) is type(other) and self.__dict__ == other.__dict__

    def __hash__(self) -> int:
        return hash((self.kind, self.index))

    def __str__(self) -> str:
        return f"{self.kind}:{self.index}"

    def __repr__(self) -> str:
        return f"{type(self).__name__}()"


class CpuDevice(Device):
    """Host memory; ``numa_node`` is recorded for the caller's own placement decisions."""

    _type = DeviceType.CPU

    def __init__(self, numa_node: Optional[int] = None):
        self.numa_node = numa_node

    def is_available(self) -> bool:
        return True

    def __repr__(self) -> str:
        return "CpuDevice()" if self.numa_node is None else f"CpuDevice(numa_node={self.numa_node})"


def _current_handle(kind: str) -> Optional[int]:
    try:
        from . import get_device_context_handle
        return get_device_context_handle(kind)
    except Exception:
        return None


class CudaDevice(Device):
    """An NVIDIA GPU by ordinal. ``context`` is kept as given; when omitted it is looked up once."""

    _type = DeviceType.CUDA

    def __init__(self, device_id: int = 0, context: Optional[int] = None):
        self.device_id = int(device_id)
        self._context = context if context is not None else _current_handle("cuda")

    def get_context_handle(self) -> Optional[int]:
        return self._context

    def is_available(self) -> bool:
        try:
            import torch
            return torch.cuda.is_available() and self.device_id < torch.cuda.device_count()
        except Exception:
            return False

    def __repr__(self) -> str:
        if self._context is not None:
            return f"CudaDevice(device_id={self.device_id}, context={self._context:#x})"
        return f"CudaDevice(device_id={self.device_id})"


class RocmDevice(Device):
    _type = DeviceType.ROCM

    def __init__(self, device_id: int = 0, context: Optional[int] = None):
        self.device_id = int(device_id)
        self._context = context if context is not None else _current_handle("rocm")

    def get_context_handle(self) -> Optional[int]:
        return self._context

    def __repr__(self) -> str:
        return f"RocmDevice(device_id={self.device_id})"


class SyclDevice(Device):
    _type = DeviceType.SYCL

    def __init__(self, device_id: int = 0, context: Optional[int] = None, queue: Optional[int] = None):
        self.device_id = int(device_id)
        self._context = context
        self.queue = queue

    def get_context_handle(self) -> Optional[int]:
        return self._context

    def __repr__(self) -> str:
        return f"SyclDevice(device_id={self.device_id})"


def cpu(numa_node: Optional[int] = None) -> CpuDevice:
    return CpuDevice(numa_node=numa_node)


def cuda(device_id: int = 0, context: Optional[int] = None) -> CudaDevice:
    return CudaDevice(device_id=device_id, context=context)


def rocm(device_id: int = 0, context: Optional[int] = None) -> RocmDevice:
    return RocmDevice(device_id=device_id, context=context)


def sycl(device_id: int = 0, context: Optional[int] = None, queue: Optional[int] = None) -> SyclDevice:
    return SyclDevice(device_id=device_id, context=context, queue=queue)


def auto_detect() -> Device:
    """A CUDA device when one is usable from this process, else the CPU."""
    d = CudaDevice(0)
    return d if d.is_available() else CpuDevice()
