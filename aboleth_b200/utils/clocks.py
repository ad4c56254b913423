"""Read-only sampling of a GPU's SM clock and throttle reasons while a measurement runs.

A benchmark number is only worth keeping with the clocks it was taken at: a thermal or hardware
slowdown, or SM clocks pinned far below the maximum, invalidates it; a software power cap during
dense tensor work is normal and only noted.  Nothing here changes a setting of the GPU.
"""
from __future__ import annotations

import statistics
import threading
from typing import Optional

_REASONS = (
    ("nvmlClocksEventReasonSwPowerCap", 0x4, "sw_power_cap"),
    ("nvmlClocksEventReasonHwSlowdown", 0x8, "hw_slowdown"),
    ("nvmlClocksEventReasonSwThermalSlowdown", 0x20, "sw_thermal_slowdown"),
    ("nvmlClocksEventReasonHwThermalSlowdown", 0x40, "hw_thermal_slowdown"),
    ("nvmlClocksEventReasonHwPowerBrakeSlowdown", 0x80, "hw_power_brake"),
)


class ClockSampler(threading.Thread):
    """Samples one GPU through NVML every ``period`` seconds between ``start()`` and ``stop()``."""

    def __init__(self, index: int, period: float = 0.1):
        super().__init__(daemon=True)
        self.index, self.period = index, period
        self.samples: list[int] = []
        self.power: list[float] = []
        self.reasons: set[str] = set()
        self.max_mhz: Optional[int] = None
        self._halt = threading.Event()
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.handle = pynvml.nvmlDeviceGetHandleByIndex(index)
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM)
        except Exception:  # noqa: BLE001
            self.nv = None

    def run(self) -> None:
        if self.nv is None:
            return
        nv = self.nv
        names = {getattr(nv, attr, bit): name for attr, bit, name in _REASONS}
        while not self._halt.is_set():
            try:
                self.samples.append(nv.nvmlDeviceGetClockInfo(self.handle, nv.NVML_CLOCK_SM))
                try:
                    self.power.append(nv.nvmlDeviceGetPowerUsage(self.handle) / 1000.0)
                except Exception:  # noqa: BLE001
                    pass
                try:
                    mask = nv.nvmlDeviceGetCurrentClocksEventReasons(self.handle)
                except Exception:  # noqa: BLE001
                    mask = nv.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle)
                for bit, name in names.items():
                    if mask & bit:
                        self.reasons.add(name)
            except Exception:  # noqa: BLE001
                pass
            self._halt.wait(self.period)

    def stop(self) -> dict:
        self._halt.set()
        if self.is_alive():
            self.join(timeout=2)
        median = statistics.median(self.samples) if self.samples else None
        return {"sm_mhz": median, "sm_max_mhz": self.max_mhz, "reasons": sorted(self.reasons),
                "samples": len(self.samples),
                "power_w_max": max(self.power) if self.power else None}
