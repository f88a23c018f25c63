"""Device timing, L2 flushing, clock sampling and roofline arithmetic."""
from __future__ import annotations

import json
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
    """Samples SM clock / power / throttle reasons with nvidia-smi while a timed
    region runs. Only reads; never changes a setting."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
             "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
             "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: List[List[str]] = []
        self._proc = None
        self._thread = None

    def start(self):
        try:
            self._proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.gpu_index}", f"--query-gpu={self.QUERY}",
                 "--format=csv,noheader,nounits", "-lms", str(self.period_ms)],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def reader():
            for line in self._proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self._thread = threading.Thread(target=reader, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> Dict:
        if self._proc is not None:
            time.sleep(self.period_ms / 1000.0)
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
                "samples": len(sm), "reasons": sorted(reasons)}
