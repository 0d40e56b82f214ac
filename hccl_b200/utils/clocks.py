"""Samples GPU clocks and throttle reasons while a timed region runs (read-only queries).

NVML is queried in-process (a few microseconds per sample, so even a 50 ms timed region yields samples); when the NVML
binding is missing, an `nvidia-smi -lms` child process is used instead. Nothing is ever set: no clocks, no power limits,
no persistence mode.
"""
from __future__ import annotations

import statistics
import subprocess
import threading
import time
from typing import Dict, List

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 5):
        self.gpu = gpu_index
        self.period = period_ms
        self.rows: List[tuple] = []            # (sm_mhz, max_mhz, set(reasons))
        self._proc = None
        self._thread = None
        self._stop = threading.Event()
        self._skip = 0

    def mark(self) -> None:
        """Samples taken so far belong to warm-up; only later ones are summarised."""
        self._skip = len(self.rows)

    # ---- NVML path ---------------------------------------------------------------------------------------------
    def _nvml_loop(self, nv, handle) -> None:
        names = (("hw_slowdown", getattr(nv, "nvmlClocksEventReasonHwSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwSlowdown", 0x8))),
                 ("hw_thermal_slowdown", getattr(nv, "nvmlClocksEventReasonHwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonHwThermalSlowdown", 0x40))),
                 ("sw_thermal_slowdown", getattr(nv, "nvmlClocksEventReasonSwThermalSlowdown", getattr(nv, "nvmlClocksThrottleReasonSwThermalSlowdown", 0x20))),
                 ("sw_power_cap", getattr(nv, "nvmlClocksEventReasonSwPowerCap", getattr(nv, "nvmlClocksThrottleReasonSwPowerCap", 0x4))))
        get_reasons = getattr(nv, "nvmlDeviceGetCurrentClocksEventReasons", None) or getattr(nv, "nvmlDeviceGetCurrentClocksThrottleReasons")
        mx = float(nv.nvmlDeviceGetMaxClockInfo(handle, nv.NVML_CLOCK_SM))
        while not self._stop.is_set():
            try:
                sm = float(nv.nvmlDeviceGetClockInfo(handle, nv.NVML_CLOCK_SM))
                mask = int(get_reasons(handle))
                self.rows.append((sm, mx, {n for n, bit in names if mask & bit}))
            except Exception:                   # noqa: BLE001 - a failed sample is skipped
                pass
            time.sleep(self.period / 1000.0)

    def start(self) -> None:
        try:
            import pynvml as nv

            nv.nvmlInit()
            handle = nv.nvmlDeviceGetHandleByIndex(self.gpu)
            self._thread = threading.Thread(target=self._nvml_loop, args=(nv, handle), daemon=True)
            self._thread.start()
            return
        except Exception:                       # noqa: BLE001 - fall back to the command line tool
            pass
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu),
                                           "-lms", str(max(self.period, 20))], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            for line in self._proc.stdout:
                r = [c.strip() for c in line.split(",")]
                if len(r) < 8:
                    continue
                try:
                    reasons = {n for n, v in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8])
                               if v.lower().startswith("active")}
                    self.rows.append((float(r[1]), float(r[2]), reasons))
                except ValueError:
                    continue

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> Dict:
        self._stop.set()
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:                   # noqa: BLE001
                pass
        if self._thread is not None:
            self._thread.join(timeout=2)
        rows = self.rows[self._skip:] or self.rows[-3:]
        if not rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        reasons = set()
        for r in rows:
            reasons |= r[2]
        return {"sm_mhz": statistics.median(r[0] for r in rows), "sm_max_mhz": max(r[1] for r in rows), "reasons": sorted(reasons), "samples": len(rows)}
