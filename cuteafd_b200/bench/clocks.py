"""GPU clock / throttle sampling during a timed region (nvidia-smi polling, read-only).

Every benchmark phase carries the clocks it ran under, as the reference attaches per-window
throttle summaries to its bench phases (rust/crates/cuteafd-core/src/thermal.rs:1-40).
"""
from __future__ import annotations

import shutil
import statistics
import subprocess

FIELDS = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
          "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
          "clocks_event_reasons.sw_power_cap")


class ClockSampler:
    def __init__(self, gpu_index: int = 0, period_ms: int = 100):
        self.gpu_index, self.period_ms = gpu_index, period_ms
        self.proc: subprocess.Popen | None = None

    def __enter__(self) -> "ClockSampler":
        exe = shutil.which("nvidia-smi")
        if exe:
            self.proc = subprocess.Popen([exe, f"--query-gpu={FIELDS}", "--format=csv,noheader,nounits",
                                          "-i", str(self.gpu_index), "-lms", str(self.period_ms)],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        return self

    def __exit__(self, *exc) -> None:
        self.lines: list[str] = []
        if self.proc is not None:
            self.proc.terminate()
            try:
                out, _ = self.proc.communicate(timeout=5)
            except subprocess.TimeoutExpired:
                self.proc.kill()
                out, _ = self.proc.communicate()
            self.lines = [l for l in out.splitlines() if l.strip()]

    def summary(self) -> dict:
        sm, mx, power, reasons = [], [], [], set()
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for line in getattr(self, "lines", []):
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2])); power.append(float(parts[3]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "power_w_max": max(power),
                "reasons": sorted(reasons), "samples": len(sm)}
