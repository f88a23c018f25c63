"""Device descriptions for AxonRuntime (same surface as the reference's
``axon/python/axon/device.py:12-299``: ``Device`` hierarchy, ``cpu() cuda() rocm()
sycl() auto_detect()``). This build drives ``cpu`` and ``cuda`` devices; the other
kinds exist so that code written against the reference imports and fails with a
clear message when such a device is actually requested."""
from __future__ import annotations

import enum
from dataclasses import dataclass


class DeviceType(enum.Enum):
    CPU = "cpu"
    CUDA = "cuda"
    ROCM = "rocm"
    SYCL = "sycl"


@dataclass(frozen=True)
class Device:
    kind: str
    index: int = 0

    @property
    def device_type(self) -> DeviceType:
        return DeviceType(self.kind)

    def is_available(self) -> bool:
        return False

    def __str__(self) -> str:
        return f"{self.kind}:{self.index}"


class CpuDevice(Device):
    def __init__(self):
        super().__init__("cpu", 0)

    def is_available(self) -> bool:
        return True


class CudaDevice(Device):
    def __init__(self, index: int = 0):
        super().__init__("cuda", index)

    def is_available(self) -> bool:
        try:
            import torch
            return torch.cuda.is_available() and self.index < torch.cuda.device_count()
        except Exception:
            return False


class RocmDevice(Device):
    def __init__(self, index: int = 0):
        super().__init__("rocm", index)


class SyclDevice(Device):
    def __init__(self, index: int = 0):
        super().__init__("sycl", index)


def cpu() -> CpuDevice:
    return CpuDevice()


def cuda(index: int = 0) -> CudaDevice:
    return CudaDevice(index)


def rocm(index: int = 0) -> RocmDevice:
    return RocmDevice(index)


def sycl(index: int = 0) -> SyclDevice:
    return SyclDevice(index)


def auto_detect() -> Device:
    """A CUDA device when one is usable, else the CPU."""
    d = cuda(0)
    return d if d.is_available() else cpu()
