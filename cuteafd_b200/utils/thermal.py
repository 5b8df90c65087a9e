"""Clock / power / temperature / throttle telemetry: a background sampler that fills a bounded ring, and window
summaries over it that a benchmark phase or ``/v1/thermal`` attaches to its numbers.

Everything here only READS the device: NVML queries (clock, power, temperature, the throttle-reason bit mask) through
``pynvml`` when it is importable, ``nvidia-smi --query-gpu`` otherwise.  No call changes a clock, a power limit or
any other setting.

    mon = ThermalMonitor(backend=open_backend(), period_s=0.2).start()
    t0 = time.monotonic(); run_phase(); t1 = time.monotonic()
    print(mon.window(t0, t1))       # {"sm_mhz": {...}, "power_w": {...}, "reasons": {"sw_power_cap": 0.93}, "verdict": ...}

A window's ``verdict`` is what decides whether a measurement stands: ``thermal`` (hardware or software thermal
slowdown seen: take the number again), ``locked`` (clocks well under the maximum with no reason active: somebody left a
clock lock), ``power_cap`` (normal for a dense GEMM on a 1 kW part: keep and note), ``ok``.

Counterpart: rust/crates/cuteafd-core/src/thermal.rs:1-40 (sampler ring, per-window throttle summaries),
rust/crates/cuteafd-daemon/src/shared/thermal.rs, rust/crates/cuteafd-ffi/src/nvml.rs (NVML bindings).
"""
from __future__ import annotations

import shutil
import statistics
import subprocess
import threading
import time
from collections import deque
from dataclasses import dataclass, field

# NVML throttle-reason bits (nvml.h: nvmlClocksEventReason*)
REASON_BITS = {
    0x0001: "gpu_idle",
    0x0002: "applications_clocks_setting",
    0x0004: "sw_power_cap",
    0x0008: "hw_slowdown",
    0x0010: "sync_boost",
    0x0020: "sw_thermal_slowdown",
    0x0040: "hw_thermal_slowdown",
    0x0080: "hw_power_brake_slowdown",
    0x0100: "display_clock_setting",
}
BAD = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "hw_power_brake_slowdown")


@dataclass
class Sample:
    t: float                      # time.monotonic()
    gpu: int
    sm_mhz: float
    sm_max_mhz: float
    mem_mhz: float = 0.0
    power_w: float = 0.0
    temp_c: float = 0.0
    reasons: int = 0              # NVML bit mask

    def reason_names(self) -> list[str]:
        return [n for b, n in REASON_BITS.items() if self.reasons & b]


class NvmlBackend:
    """Reads through an NVML module object (``pynvml`` or a stand-in with the same functions)."""

    def __init__(self, nvml, gpus: list[int] | None = None):
        self.nvml = nvml
        nvml.nvmlInit()
        n = nvml.nvmlDeviceGetCount()
        self.gpus = list(range(n)) if gpus is None else [g for g in gpus if g < n]
        self.handles = {g: nvml.nvmlDeviceGetHandleByIndex(g) for g in self.gpus}

    def read(self) -> list[Sample]:
        nv, out, now = self.nvml, [], time.monotonic()
        for g, h in self.handles.items():
            try:
                out.append(Sample(now, g,
                                  float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)),
                                  float(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM)),
                                  float(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_MEM)),
                                  nv.nvmlDeviceGetPowerUsage(h) / 1000.0,
                                  float(nv.nvmlDeviceGetTemperature(h, nv.NVML_TEMPERATURE_GPU)),
                                  int(nv.nvmlDeviceGetCurrentClocksThrottleReasons(h))))
            except Exception:                                      # noqa: BLE001 - a failed query drops the sample, not the monitor
                continue
        return out

    def close(self) -> None:
        try:
            self.nvml.nvmlShutdown()
        except Exception:                                          # noqa: BLE001
            pass


class SmiBackend:
    """One ``nvidia-smi`` query per read (slower; used when NVML bindings are missing)."""
    FIELDS = ("index,clocks.sm,clocks.max.sm,clocks.mem,power.draw,temperature.gpu,clocks_event_reasons.sw_power_cap,"
              "clocks_event_reasons.hw_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown")
    _BITS = (0x0004, 0x0008, 0x0020, 0x0040)

    def __init__(self, exe: str | None = None, run=None):
        self.exe = exe or shutil.which("nvidia-smi")
        self.run = run or self._run

    def _run(self) -> str:
        if not self.exe:
            return ""
        try:
            return subprocess.run([self.exe, f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits"],
                                  capture_output=True, text=True, timeout=5).stdout
        except (OSError, subprocess.TimeoutExpired):
            return ""

    def read(self) -> list[Sample]:
        out, now = [], time.monotonic()
        for line in self.run().splitlines():
            p = [x.strip() for x in line.split(",")]
            if len(p) < 10:
                continue
            try:
                mask = 0
                for bit, v in zip(self._BITS, p[6:10]):
                    if v.lower().startswith("active"):
                        mask |= bit
                out.append(Sample(now, int(p[0]), float(p[1]), float(p[2]), float(p[3]), float(p[4]), float(p[5]), mask))
            except ValueError:
                continue
        return out

    def close(self) -> None:
        pass


def open_backend(gpus: list[int] | None = None):
    """NVML when its bindings import and initialise, else nvidia-smi, else None (no GPU on this host)."""
    try:
        import pynvml
        return NvmlBackend(pynvml, gpus)
    except Exception:                                              # noqa: BLE001
        pass
    return SmiBackend() if shutil.which("nvidia-smi") else None


def _stats(xs: list[float]) -> dict:
    if not xs:
        return {"median": None, "min": None, "max": None}
    return {"median": statistics.median(xs), "min": min(xs), "max": max(xs)}


def summarize(samples: list[Sample], lock_ratio: float = 0.75) -> dict:
    """Summary of one GPU's samples of one window."""
    if not samples:
        return {"samples": 0, "verdict": "unmeasured", "reasons": {}}
    n = len(samples)
    frac: dict[str, float] = {}
    for s in samples:
        for name in s.reason_names():
            frac[name] = frac.get(name, 0) + 1
    frac = {k: round(v / n, 3) for k, v in sorted(frac.items()) if k != "gpu_idle"}
    sm = _stats([s.sm_mhz for s in samples])
    mx = max(s.sm_max_mhz for s in samples)
    busy = [s for s in samples if not s.reasons & 0x0001]
    verdict = "ok"
    if any(k in frac for k in BAD):
        verdict = "thermal"
    elif busy and mx and statistics.median(s.sm_mhz for s in busy) < lock_ratio * mx and not any(
            s.reasons & ~0x0001 for s in busy):
        verdict = "locked"
    elif "sw_power_cap" in frac:
        verdict = "power_cap"
    return {"samples": n, "seconds": round(samples[-1].t - samples[0].t, 3), "sm_mhz": sm, "sm_max_mhz": mx,
            "mem_mhz": _stats([s.mem_mhz for s in samples]), "power_w": _stats([s.power_w for s in samples]),
            "temp_c": _stats([s.temp_c for s in samples]), "reasons": frac, "verdict": verdict}


@dataclass
class ThermalMonitor:
    backend: object = None
    period_s: float = 0.2
    capacity: int = 18000                                         # an hour at 5 Hz per GPU
    ring: dict[int, deque] = field(default_factory=dict)

    def __post_init__(self) -> None:
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None
        self._lock = threading.Lock()

    # ---- sampling -------------------------------------------------------------------------
    def poll(self) -> int:
        """Take one reading now (the thread's body; tests call it directly)."""
        if self.backend is None:
            return 0
        got = self.backend.read()
        with self._lock:
            for s in got:
                self.ring.setdefault(s.gpu, deque(maxlen=self.capacity)).append(s)
        return len(got)

    def start(self) -> "ThermalMonitor":
        if self.backend is None or self._thread is not None:
            return self

        def loop() -> None:
            while not self._stop.wait(self.period_s):
                self.poll()
        self.poll()
        self._thread = threading.Thread(target=loop, name="thermal-sampler", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)
            self._thread = None
        if self.backend is not None:
            self.backend.close()

    # ---- queries --------------------------------------------------------------------------
    def latest(self) -> dict:
        with self._lock:
            return {g: vars(r[-1]) | {"reason_names": r[-1].reason_names()} for g, r in self.ring.items() if r}

    def window(self, t0: float, t1: float | None = None, gpu: int | None = None) -> dict:
        """Summary of the samples with t0 <= t <= t1 (monotonic clock), per GPU or for one GPU."""
        t1 = time.monotonic() if t1 is None else t1
        with self._lock:
            picked = {g: [s for s in r if t0 <= s.t <= t1] for g, r in self.ring.items()}
        if gpu is not None:
            return summarize(picked.get(gpu, []))
        return {g: summarize(v) for g, v in sorted(picked.items())}

    def report(self, seconds: float = 60.0) -> dict:
        now = time.monotonic()
        return {"available": self.backend is not None, "latest": self.latest(), "window_seconds": seconds,
                "window": self.window(now - seconds, now)}


_GLOBAL: ThermalMonitor | None = None


def monitor() -> ThermalMonitor:
    """The process-wide monitor (started on first use)."""
    global _GLOBAL
    if _GLOBAL is None:
        _GLOBAL = ThermalMonitor(open_backend()).start()
    return _GLOBAL


def sample_once() -> dict:
    """One reading without a background thread (``/v1/thermal`` on a server that runs no monitor)."""
    be = open_backend()
    if be is None:
        return {"available": False}
    got = be.read()
    be.close()
    return {"available": True, "gpus": [vars(s) | {"reason_names": s.reason_names()} for s in got]}
