"""Samples GPU clocks and throttle reasons with nvidia-smi while a timed region runs (read-only queries)."""
from __future__ import annotations

import statistics
import subprocess
import threading
from typing import Dict, List

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
           "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 50):
        self.gpu = gpu_index
        self.period = period_ms
        self.rows: List[List[str]] = []
        self._proc = None
        self._thread = None
        self._skip = 0

    def mark(self) -> None:
        """Samples taken so far belong to warm-up; only later ones are summarised."""
        self._skip = len(self.rows)

    def start(self) -> None:
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu),
                                           "-lms", str(self.period)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return

        def pump():
            for line in self._proc.stdout:
                self.rows.append([c.strip() for c in line.split(",")])

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()

    def stop(self) -> Dict:
        if self._proc is not None:
            self._proc.terminate()
            try:
                self._proc.wait(timeout=5)
            except Exception:
                pass
        sm, mx, reasons = [], [], set()
        rows = self.rows[self._skip:] or self.rows[-3:]
        for r in rows:
            if len(r) < 8:
                continue
            try:
                sm.append(float(r[1]))
                mx.append(float(r[2]))
            except ValueError:
                continue
            for name, val in zip(("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"), r[4:8]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}
