"""Memory ledger: every long-lived device allocation is tagged (kind, owner); the ledger can be
reconciled against what the allocator reports.  Counterpart:
rust/crates/cuteafd-ffi/src/memory_ledger.rs:1-60, rust/crates/cuteafd-daemon/src/shared/memory_report.rs.
"""
from __future__ import annotations

import threading


class MemoryLedger:
    def __init__(self) -> None:
        self.entries: dict[tuple[str, str], int] = {}
        self.lock = threading.Lock()

    def tag(self, kind: str, owner: str, nbytes: int) -> None:
        with self.lock:
            self.entries[(kind, owner)] = self.entries.get((kind, owner), 0) + int(nbytes)

    def tag_tensor(self, kind: str, owner: str, t) -> None:
        self.tag(kind, owner, t.numel() * t.element_size())

    def release(self, kind: str, owner: str) -> None:
        with self.lock:
            self.entries.pop((kind, owner), None)

    def total(self) -> int:
        return sum(self.entries.values())

    def report(self) -> dict:
        by_kind: dict[str, int] = {}
        for (k, _), v in self.entries.items():
            by_kind[k] = by_kind.get(k, 0) + v
        out = {"tracked_bytes": self.total(), "by_kind": by_kind,
               "entries": [{"kind": k, "owner": o, "bytes": v} for (k, o), v in sorted(self.entries.items())]}
        try:
            import torch
            if torch.cuda.is_available():
                free, total = torch.cuda.mem_get_info()
                out["device"] = {"free": free, "total": total, "torch_allocated": torch.cuda.memory_allocated(),
                                 "untracked": torch.cuda.memory_allocated() - self.total()}
        except Exception:                                   # noqa: BLE001
            pass
        return out


LEDGER = MemoryLedger()
