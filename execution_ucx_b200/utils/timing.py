"""Device timing, L2 flushing, clock sampling and roofline arithmetic."""
from __future__ import annotations

import json
import os
import statistics
import subprocess
import threading
import time
from pathlib import Path
from typing import Callable, Dict, List, Optional

import torch

_ROOT = Path(__file__).resolve().parent.parent.parent

FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0, "source": "fallback"}
NVLINK_PEER_GBS = 770.0      # measured peer copy, per direction per GPU
NVLINK_NOMINAL_GBS = 900.0


def measured_peaks() -> Dict[str, float]:
    """Roofline denominators: the driver-written measurement, else the stated fallback."""
    p = _ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        d["source"] = "measured"
        return d
    return dict(FALLBACK_PEAKS)


class L2Flusher:
    """Writes a buffer larger than L2 (126 MB) between timed iterations."""

    def __init__(self, device, nbytes: int = 256 << 20):
        self.buf = torch.empty(nbytes, dtype=torch.uint8, device=device)

    def __call__(self):
        self.buf.zero_()


def time_cuda(fn: Callable[[], None], iters: int, warmup: int = 3, flush: Optional[L2Flusher] = None,
              before: Optional[Callable[[], None]] = None) -> List[float]:
    """Per-iteration device time in ms: CUDA events on the launching stream,
    synchronize on both sides, optional L2 flush (untimed) before each iteration."""
    for _ in range(warmup):
        if before:
            before()
        fn()
    torch.cuda.synchronize()
    out = []
    for _ in range(iters):
        if flush:
            flush()
        if before:
            before()
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        a.record()
        fn()
        b.record()
        torch.cuda.synchronize()
        out.append(a.elapsed_time(b))
    return out


def percentile(xs: List[float], q: float) -> float:
    s = sorted(xs)
    if not s:
        return float("nan")
    k = min(len(s) - 1, max(0, int(round(q / 100.0 * (len(s) - 1)))))
    return s[k]


class ClockSampler:
    """Samples SM clock, power and throttle reasons while a timed region runs: through NVML from a
    thread of this process (10 ms period by default), or through an `nvidia-smi -lms` child when NVML cannot be loaded. Only reads; never
    changes a setting."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")
    REASON_BITS = {"sw_power_cap": 0x4, "hw_slowdown": 0x8, "sw_thermal_slowdown": 0x20, "hw_thermal_slowdown": 0x40}

    def __init__(self, gpu_index: int = 0, period_ms: Optional[float] = None):
        # EUX_CLOCK_PERIOD_MS overrides the period; queries take driver locks, so a very short
        # period can delay the launches it is meant to observe
        if period_ms is None:
            period_ms = float(os.environ.get("EUX_CLOCK_PERIOD_MS", "10"))
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: List[List[str]] = []
        self._proc = None
        self._thread = None
        self._stop = threading.Event()
        self._sm: List[float] = []
        self._power: List[float] = []
        self._max = None
        self._reasons = set()
        self._source = None

    def _nvml_handle(self):
        import pynvml
        pynvml.nvmlInit()
        try:
            import torch
            uuid = str(torch.cuda.get_device_properties(self.gpu_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            return pynvml, pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
        except Exception:
            return pynvml, pynvml.nvmlDeviceGetHandleByIndex(self.gpu_index)

    def start(self):
        try:
            nv, h = self._nvml_handle()
            self._max = float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            reasons_fn = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or nv.nvmlDeviceGetCurrentClocksThrottleReasons

            def loop():
                while not self._stop.is_set():
                    try:
                        self._sm.append(float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                        bits = int(reasons_fn(h))
                        for name, bit in self.REASON_BITS.items():
                            if bits & bit:
                                self._reasons.add(name)
                        self._power.append(nv.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    except Exception:
                        pass
                    self._stop.wait(self.period_ms / 1000.0)

            self._source = "nvml"
            self._thread = threading.Thread(target=loop, daemon=True)
            self._thread.start()
            return self
        except Exception:
            self._source = None
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", str(max(10, int(self.period_ms)))],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self
        self._source = "nvidia-smi"

        def reader():
            for line in self._proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self._thread = threading.Thread(target=reader, daemon=True)
        self._thread.start()
        return self

    def mark(self) -> None:
        """Forget what was sampled so far: the timed region starts here."""
        self._sm.clear()
        self._power.clear()
        self._reasons.clear()
        self.rows.clear()

    def stop(self) -> Dict:
        if self._source == "nvml":
            self._stop.set()
            self._thread.join(timeout=2)
            return {"sm_mhz": statistics.median(self._sm) if self._sm else None, "sm_max_mhz": self._max,
                    "samples": len(self._sm), "reasons": sorted(self._reasons),
                    "power_w_median": round(statistics.median(self._power), 1) if self._power else None, "source": "nvml"}
        if self._proc is not None:
            time.sleep(0.05)
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                self._proc.kill()
            if self._thread:
                self._thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            try:
                sm.append(float(r[1])), mx.append(float(r[2]))
            except (ValueError, IndexError):
                continue
            for n, v in zip(names, r[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "samples": len(sm), "reasons": sorted(reasons), "source": "nvidia-smi"}


