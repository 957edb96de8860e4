"""Read-only sampling of a GPU's SM clock, power draw and throttle reasons through NVML while a benchmark runs.

A number measured while ``hw_slowdown`` or a thermal slowdown was active, or with the SM clock pinned far below its
maximum for no stated reason, does not describe the kernel; ``sw_power_cap`` during dense GEMMs is normal on a 1 kW part
and is only noted. Nothing here changes a setting of the GPU.
"""
from __future__ import annotations

import os
import threading
import time


class ClockSampler(threading.Thread):
    """``s = ClockSampler(index); s.start(); ...; summary = s.stop()``. ``mark()`` returns the number of samples taken
    so far, so that a caller can cut the record into phases (``summary_between``)."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown",
               0x80: "hw_power_brake"}

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples, self.power, self.masks = [], [], []
        self.max_mhz = None
        self._halt = threading.Event()
        self.ok = False

    def run(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM)
            self.ok = True
            while not self._halt.is_set():
                self.samples.append(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM))
                try:
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                except Exception:
                    self.power.append(0.0)
                self.masks.append(int(pynvml.nvmlDeviceGetCurrentClocksEventReasons(h)))
                time.sleep(self.period)
        except Exception:
            self.ok = False

    def mark(self) -> int:
        return len(self.samples)

    def summary_between(self, a: int, b: int) -> dict:
        s = sorted(self.samples[a:b])
        p = sorted(self.power[a:b])
        reasons = set()
        for m in self.masks[a:b]:
            for bit, name in self.REASONS.items():
                if m & bit:
                    reasons.add(name)
        return {"sm_mhz": s[len(s) // 2] if s else None, "sm_max_mhz": self.max_mhz,
                "power_w": round(p[len(p) // 2], 1) if p else None, "reasons": sorted(reasons), "samples": len(s)}

    def stop(self) -> dict:
        self._halt.set()
        self.join(timeout=2)
        return self.summary_between(0, len(self.samples))


def visible_index(local_rank: int) -> int:
    """NVML index of the CUDA device ``local_rank`` of this process (honours CUDA_VISIBLE_DEVICES given as indices)."""
    vis = os.environ.get("CUDA_VISIBLE_DEVICES")
    if vis:
        try:
            return int(vis.split(",")[local_rank])
        except Exception:
            return local_rank
    return local_rank
