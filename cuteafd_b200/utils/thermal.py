"""Clock / power / throttle telemetry (read-only NVML or nvidia-smi sampling).

Counterpart: rust/crates/cuteafd-core/src/thermal.rs:1-40, rust/crates/cuteafd-ffi/src/nvml.rs.
Nothing here changes a GPU setting.
"""
from __future__ import annotations

import shutil
import subprocess

from ..bench.clocks import FIELDS


def sample_once() -> dict:
    exe = shutil.which("nvidia-smi")
    if not exe:
        return {"available": False}
    try:
        out = subprocess.run([exe, f"--query-gpu={FIELDS}", "--format=csv,noheader,nounits"], capture_output=True, text=True, timeout=5).stdout
    except (OSError, subprocess.TimeoutExpired):
        return {"available": False}
    gpus = []
    for line in out.splitlines():
        p = [x.strip() for x in line.split(",")]
        if len(p) >= 9:
            gpus.append({"index": p[0], "sm_mhz": p[1], "sm_max_mhz": p[2], "power_w": p[3],
                         "throttle": {k: v for k, v in zip(("hw_slowdown", "hw_thermal", "sw_thermal", "sw_power_cap"), p[5:9])}})
    return {"available": True, "gpus": gpus}
