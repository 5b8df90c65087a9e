"""``cuteafd doctor``: environment checks (toolchain, native libraries, GPU visibility)."""
from __future__ import annotations

import shutil


def doctor() -> tuple[bool, list[str]]:
    lines, ok = [], True
    import torch
    lines.append(f"torch {torch.__version__}, cuda available: {torch.cuda.is_available()}")
    nvcc = shutil.which("nvcc") or "/usr/local/cuda/bin/nvcc"
    lines.append(f"nvcc: {nvcc if shutil.which(nvcc) or __import__('os').path.exists(nvcc) else 'MISSING'}")
    try:
        from .._native import lib
        lib.cuda_lib()
        lines.append("libcuteafd_b200.so: loaded")
    except Exception as e:                                 # noqa: BLE001
        ok = False
        lines.append(f"libcuteafd_b200.so: FAILED ({e})")
    try:
        from .._native import lib
        lib.rt_lib()
        lines.append("libcuteafd_rt.so: loaded")
    except Exception as e:                                 # noqa: BLE001
        lines.append(f"libcuteafd_rt.so: not loaded ({e})")
    if torch.cuda.is_available():
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            good = (p.major, p.minor) == (10, 0)
            ok &= good
            lines.append(f"gpu{i}: {p.name} sm_{p.major}{p.minor} {'ok' if good else 'NOT sm_100'}")
    return ok, lines
