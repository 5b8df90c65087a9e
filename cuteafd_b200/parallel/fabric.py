"""NVLink / peer-access report for ``cuteafd fabric`` and ``/v1/fabric`` (read-only queries).

Counterpart: rust/crates/cuteafd-transport/src/fabric.rs, fabric_health.rs and the ``fabric``
subcommand (rust/crates/cuteafd-daemon/src/cli.rs:297-340); RoCE rails become NVLink peers.
"""
from __future__ import annotations


def fabric_report(p2p: bool = False) -> dict:
    import torch
    out: dict = {"cuda": torch.cuda.is_available(), "devices": []}
    if not torch.cuda.is_available():
        return out
    n = torch.cuda.device_count()
    for i in range(n):
        pr = torch.cuda.get_device_properties(i)
        out["devices"].append({"index": i, "name": pr.name, "sms": pr.multi_processor_count, "memory_gib": round(pr.total_memory / 2**30, 1),
                               "capability": f"{pr.major}.{pr.minor}"})
    out["peer_access"] = [[(i == j) or torch.cuda.can_device_access_peer(i, j) for j in range(n)] for i in range(n)]
    if p2p and n >= 2:
        a = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:0")
        b = torch.empty(256 << 20, dtype=torch.uint8, device="cuda:1")
        for _ in range(2):
            b.copy_(a)
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record(); b.copy_(a); e.record(); torch.cuda.synchronize()
        out["p2p_copy_gbs_0_to_1"] = round(a.numel() / s.elapsed_time(e) / 1e6, 1)
    return out
