"""Device-side timing and clock sampling.

The reference times GPU work with os.clock() and no device synchronise
(tools/benchmark.lua:14-27), which measures launch cost.  `DeviceTimer` brackets a region with
CUDA events on the launching stream; `ClockSampler` records SM clocks and throttle reasons
through NVML (read-only queries) while a timed region runs."""
from __future__ import annotations

import statistics
import threading
import time
from typing import List, Optional

import torch


class DeviceTimer:
    def __init__(self):
        self.start = torch.cuda.Event(enable_timing=True)
        self.stop = torch.cuda.Event(enable_timing=True)

    def __enter__(self):
        torch.cuda.synchronize()
        self.start.record()
        return self

    def __exit__(self, *exc):
        self.stop.record()
        torch.cuda.synchronize()
        self.ms = self.start.elapsed_time(self.stop)
        return False


_REASONS = {
    0x1: "gpu_idle", 0x2: "applications_clocks_setting", 0x4: "sw_power_cap", 0x8: "hw_slowdown",
    0x10: "sync_boost", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
    0x80: "hw_power_brake_slowdown", 0x100: "display_clock_setting",
}


class ClockSampler:
    """Samples SM clock / throttle reasons of one GPU every `period_s` in a host thread."""

    def __init__(self, device_index: int = 0, period_s: float = 0.1):
        self.device_index = device_index
        self.period_s = period_s
        self.samples: List[int] = []
        self.reasons = set()
        self.max_mhz: Optional[int] = None
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._ok = False
        try:
            import pynvml
            pynvml.nvmlInit()
            self._nv = pynvml
            self._h = pynvml.nvmlDeviceGetHandleByIndex(device_index)
            self.max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._h, pynvml.NVML_CLOCK_SM))
            self._ok = True
        except Exception:
            self._ok = False

    def _run(self):
        nv = self._nv
        while not self._stop.is_set():
            try:
                self.samples.append(int(nv.nvmlDeviceGetClockInfo(self._h, nv.NVML_CLOCK_SM)))
                mask = int(nv.nvmlDeviceGetCurrentClocksEventReasons(self._h))
                for bit, name in _REASONS.items():
                    if mask & bit and name != "gpu_idle":
                        self.reasons.add(name)
            except Exception:
                pass
            time.sleep(self.period_s)

    def start(self):
        if self._ok:
            self._thread = threading.Thread(target=self._run, daemon=True)
            self._thread.start()
        return self

    def stop(self) -> dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2.0)
        med = int(statistics.median(self.samples)) if self.samples else None
        return {"sm_mhz": med, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples)}
