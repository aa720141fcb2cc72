"""Read-only sampling of SM clocks and throttle reasons while a timed region runs (NVML through
``pynvml``; falls back to parsing ``nvidia-smi``).  Nothing here changes a GPU setting."""
from __future__ import annotations

import subprocess
import threading
import time
from typing import Dict, List, Optional

_REASONS = {  # NVML clocks-event-reason bits
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000080: "hw_power_brake_slowdown",
}


class ClockSampler:
    def __init__(self, gpu_index: int, period_s: float = 0.01):
        self.gpu_index, self.period_s = gpu_index, period_s
        self.sm: List[float] = []
        self.power: List[float] = []
        self.sm_max: Optional[float] = None
        self.reasons = set()
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._how = "none"

    def _physical_index(self) -> int:
        import os
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            try:
                return int(vis.split(",")[self.gpu_index])
            except (ValueError, IndexError):
                pass
        return self.gpu_index

    def _run_nvml(self) -> bool:
        try:
            import pynvml
            pynvml.nvmlInit()
            h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.sm_max = float(pynvml.nvmlDeviceGetMaxClockInfo(h, pynvml.NVML_CLOCK_SM))
        except Exception:  # noqa: BLE001
            return False
        self._how = "nvml"

        def loop():
            get_reasons = getattr(pynvml, "nvmlDeviceGetCurrentClocksEventReasons", None) or \
                getattr(pynvml, "nvmlDeviceGetCurrentClocksThrottleReasons", None)
            while not self._stop.is_set():
                try:
                    self.sm.append(float(pynvml.nvmlDeviceGetClockInfo(h, pynvml.NVML_CLOCK_SM)))
                    self.power.append(pynvml.nvmlDeviceGetPowerUsage(h) / 1000.0)
                    if get_reasons is not None:
                        bits = int(get_reasons(h))
                        for bit, name in _REASONS.items():
                            if bits & bit:
                                self.reasons.add(name)
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(self.period_s)
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()
        return True

    def _run_smi(self) -> None:
        self._how = "nvidia-smi"
        fields = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
                  "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
                  "clocks_event_reasons.sw_power_cap")

        def loop():
            while not self._stop.is_set():
                try:
                    out = subprocess.run(["nvidia-smi", f"--id={self._physical_index()}", f"--query-gpu={fields}",
                                          "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
                    parts = [p.strip() for p in out.strip().split(",")]
                    self.sm.append(float(parts[0])); self.sm_max = float(parts[1]); self.power.append(float(parts[2]))
                    for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), parts[3:7]):
                        if val.lower().startswith("active"):
                            self.reasons.add(name)
                except Exception:  # noqa: BLE001
                    pass
                time.sleep(max(self.period_s, 0.2))
        self._thread = threading.Thread(target=loop, daemon=True)
        self._thread.start()

    def start(self) -> "ClockSampler":
        if not self._run_nvml():
            self._run_smi()
        return self

    def stop(self) -> Dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=6)
        sm = sorted(self.sm)
        return {"sm_mhz": sm[len(sm) // 2] if sm else None, "sm_max_mhz": self.sm_max,
                "power_w_max": max(self.power) if self.power else None, "samples": len(sm),
                "reasons": sorted(self.reasons), "source": self._how}
