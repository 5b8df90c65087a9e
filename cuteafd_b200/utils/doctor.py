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
    # host pieces every deployment relies on
    try:
        from ..runtime.native import NativeRepeatGuard, wire_crc32
        from ..runtime.repeat_guard import LoopAbortConfig
        NativeRepeatGuard(LoopAbortConfig()).push(1)
        import zlib
        good = wire_crc32(b"doctor") == zlib.crc32(b"doctor")
        ok &= good
        lines.append(f"runtime twins (loop guard, wire headers): {'ok' if good else 'MISMATCH'}")
    except Exception as e:                                 # noqa: BLE001
        ok = False
        lines.append(f"runtime twins: FAILED ({e})")
    from .thermal import open_backend
    be = open_backend()
    if be is None:
        lines.append("telemetry: no NVML bindings and no nvidia-smi (thermal endpoints will report unavailable)")
    else:
        got = be.read()
        be.close()
        lines.append(f"telemetry: {type(be).__name__}, {len(got)} GPU(s) readable" +
                     ("".join(f"; gpu{s.gpu} {int(s.sm_mhz)}/{int(s.sm_max_mhz)} MHz {','.join(s.reason_names()) or 'no throttle reason'}" for s in got[:8])))
    for mod in ("safetensors", "tokenizers", "numpy"):
        try:
            __import__(mod)
            lines.append(f"{mod}: importable")
        except ImportError:
            lines.append(f"{mod}: not installed" + (" (byte tokenizer only)" if mod == "tokenizers" else " (built-in reader is used)" if mod == "safetensors" else ""))
    if torch.cuda.is_available():
        n = torch.cuda.device_count()
        if n > 1:
            missing = [(i, j) for i in range(n) for j in range(n) if i != j and not torch.cuda.can_device_access_peer(i, j)]
            ok &= not missing
            lines.append("peer access: every pair" if not missing else f"peer access MISSING for {missing[:6]} (the exchange needs it)")
        for i in range(torch.cuda.device_count()):
            p = torch.cuda.get_device_properties(i)
            good = (p.major, p.minor) == (10, 0)
            ok &= good
            lines.append(f"gpu{i}: {p.name} sm_{p.major}{p.minor} {'ok' if good else 'NOT sm_100'}")
    return ok, lines
