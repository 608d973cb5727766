"""Sample SM clock, power and throttle reasons of one GPU while a benchmark runs.

Read-only: nothing here changes a clock, a power limit or any other device setting.
Sampling uses NVML through ``pynvml`` when present, else an ``nvidia-smi`` query loop.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Dict, List, Optional

_REASON_BITS = {
    0x0000000000000004: "sw_power_cap",
    0x0000000000000008: "hw_slowdown",
    0x0000000000000020: "sw_thermal_slowdown",
    0x0000000000000040: "hw_thermal_slowdown",
    0x0000000000000080: "hw_power_brake_slowdown",
}


class ClockSampler:
    def __init__(self, device_index: int = 0, period_s: float = 0.2):
        self.index = device_index
        self.period = period_s
        self.samples: List[Dict] = []
        self._stop = threading.Event()
        self._thread: Optional[threading.Thread] = None
        self._nvml = None
        self.sm_max_mhz: Optional[int] = None

    def _open_nvml(self) -> bool:
        try:
            import pynvml

            pynvml.nvmlInit()
            self._nvml = pynvml
            self._handle = pynvml.nvmlDeviceGetHandleByIndex(self.index)
            self.sm_max_mhz = int(pynvml.nvmlDeviceGetMaxClockInfo(self._handle, pynvml.NVML_CLOCK_SM))
            return True
        except Exception:  # noqa: BLE001
            self._nvml = None
            return False

    def _sample_nvml(self) -> Dict:
        n = self._nvml
        sm = int(n.nvmlDeviceGetClockInfo(self._handle, n.NVML_CLOCK_SM))
        try:
            power = n.nvmlDeviceGetPowerUsage(self._handle) / 1000.0
        except Exception:  # noqa: BLE001
            power = None
        try:
            bits = int(n.nvmlDeviceGetCurrentClocksEventReasons(self._handle))
        except Exception:  # noqa: BLE001
            try:
                bits = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self._handle))
            except Exception:  # noqa: BLE001
                bits = 0
        reasons = [name for bit, name in _REASON_BITS.items() if bits & bit]
        return {"sm_mhz": sm, "power_w": power, "reasons": reasons}

    def _sample_smi(self) -> Optional[Dict]:
        q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")
        try:
            out = subprocess.run(["nvidia-smi", f"--id={self.index}", f"--query-gpu={q}", "--format=csv,noheader,nounits"],
                                 capture_output=True, text=True, timeout=5).stdout.strip().split(",")
            self.sm_max_mhz = int(float(out[1]))
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            reasons = [n for n, v in zip(names, out[3:7]) if v.strip().lower() == "active"]
            return {"sm_mhz": int(float(out[0])), "power_w": float(out[2]), "reasons": reasons}
        except Exception:  # noqa: BLE001
            return None

    def _run(self) -> None:
        use_nvml = self._open_nvml()
        while not self._stop.is_set():
            try:
                s = self._sample_nvml() if use_nvml else self._sample_smi()
            except Exception:  # noqa: BLE001
                s = None
            if s is not None:
                self.samples.append(s)
            self._stop.wait(self.period)

    def start(self) -> "ClockSampler":
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> Dict:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=5)
        return self.summary()

    def summary(self) -> Dict:
        if not self.samples:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max_mhz, "reasons": [], "samples": 0}
        clocks = [s["sm_mhz"] for s in self.samples]
        reasons = sorted({r for s in self.samples for r in s["reasons"]})
        powers = [s["power_w"] for s in self.samples if s["power_w"] is not None]
        return {
            "sm_mhz": int(statistics.median(clocks)),
            "sm_max_mhz": self.sm_max_mhz,
            "reasons": reasons,
            "samples": len(clocks),
            "power_w_max": max(powers) if powers else None,
        }
