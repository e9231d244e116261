"""Samples SM clocks and throttle reasons with nvidia-smi while a timed region runs
(read-only queries; nothing about the GPU is changed)."""
from __future__ import annotations

import statistics
import subprocess
import threading

_FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
           "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 200):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.rows: list[list[str]] = []
        self._proc = None
        self._thread = None

    def start(self) -> "ClockSampler":
        try:
            self._proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={_FIELDS}", "--format=csv,noheader,nounits", "-i", str(self.gpu_index),
                                           "-lms", str(self.period_ms)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self._proc = None
            return self

        def pump():
            for line in self._proc.stdout:
                parts = [p.strip() for p in line.split(",")]
                if len(parts) >= 9:
                    self.rows.append(parts)

        self._thread = threading.Thread(target=pump, daemon=True)
        self._thread.start()
        return self

    def stop(self) -> dict:
        if self._proc is not None:
            self._proc.terminate()      # this exact child, nothing else
            try:
                self._proc.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self._proc.kill()
        sm = []
        for r in self.rows:
            try:
                sm.append(float(r[1]))
            except ValueError:
                pass
        reasons = set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            for name, val in zip(names, r[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        sm_max = None
        for r in self.rows:
            try:
                sm_max = float(r[2])
                break
            except ValueError:
                pass
        # under load = upper half of the samples (idle samples before/after the region are excluded)
        busy = sorted(sm)[len(sm) // 2:] if sm else []
        return {"sm_mhz": statistics.median(busy) if busy else None, "sm_max_mhz": sm_max, "reasons": sorted(reasons), "samples": len(sm)}
