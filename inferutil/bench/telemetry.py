"""GPU telemetry sources for the timed decode window (reference: src/inferutil/bench/telemetry.py:9-97).
``NvmlTelemetry`` polls NVML from a daemon thread (read-only queries); without NVML it reports unavailable."""
from __future__ import annotations

import threading
import time
from dataclasses import dataclass
from typing import List, Protocol


@dataclass(frozen=True)
class GpuSample:
    gpu_index: int
    t_seconds: float
    temp_c: float
    sm_util_pct: float
    mem_util_pct: float
    power_w: float
    sm_clock_mhz: float
    mem_clock_mhz: float
    mem_used_bytes: int


class TelemetrySource(Protocol):
    available: bool

    def start(self) -> None: ...
    def stop(self) -> list: ...


class NullTelemetry:
    available = False

    def start(self) -> None:
        return None

    def stop(self) -> list:
        return []


class FakeTelemetrySource:
    """Replays canned samples (tests)."""

    def __init__(self, samples):
        self.available = True
        self._samples = list(samples)

    def start(self) -> None:
        return None

    def stop(self) -> list:
        return self._samples


class NvmlTelemetry:
    def __init__(self, interval_s: float = 0.05):
        self.interval_s = interval_s
        self._samples: List[GpuSample] = []
        self._halt = threading.Event()
        self._thread = None
        self._nvml = None
        self._count = 0
        self.available = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nvml, self._count = pynvml, pynvml.nvmlDeviceGetCount()
            self.available = True
        except Exception:
            pass

    def _poll(self, t0: float) -> None:
        nv = self._nvml
        handles = [nv.nvmlDeviceGetHandleByIndex(i) for i in range(self._count)]
        while not self._halt.is_set():
            now = time.monotonic() - t0
            for i, h in enumerate(handles):
                util = nv.nvmlDeviceGetUtilizationRates(h)
                self._samples.append(GpuSample(
                    i, now, float(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU)), float(util.gpu),
                    float(util.memory), nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                    float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                    float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_MEM)), int(nv.nvmlDeviceGetMemoryInfo(h).used)))
            self._halt.wait(self.interval_s)

    def start(self) -> None:
        if not self.available:
            return
        self._samples = []
        self._halt.clear()
        self._thread = threading.Thread(target=self._poll, args=(time.monotonic(),), daemon=True)
        self._thread.start()

    def stop(self) -> list:
        if not self.available:
            return []
        self._halt.set()
        if self._thread is not None:
            self._thread.join(timeout=1.0)
        return list(self._samples)
