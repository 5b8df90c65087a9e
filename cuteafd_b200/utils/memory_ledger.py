"""Memory ledger: every long-lived device allocation is tagged (kind, owner, device); the ledger is reconciled against
what the driver reports, printed on a period, and dumped to a spool file that was opened at start-up when an
allocation fails (by then the process may be unable to open files or format large strings).

    LEDGER.tag_tree("weights", "engine", engine.W)          # walks dataclasses / dicts / lists for tensors
    LEDGER.tag_tree("kv", "engine", engine.cache)
    print(LEDGER.report())                                   # tracked by kind, device free/total, untracked bytes
    with LEDGER.guard("prefill workspace"):                  # OutOfMemory inside -> dump, then re-raise
        ...

Kinds are free strings; the ones the engines use are ``weights``, ``kv``, ``workspace``, ``graphs``, ``exchange``
(symmetric buffers other GPUs write into), ``media``.  Tensors that share storage are counted once.

Counterpart: rust/crates/cuteafd-ffi/src/memory_ledger.rs:1-60 (tagged allocations), memory_ledger/fault.rs:1-20
(failure spool opened at start-up), rust/crates/cuteafd-daemon/src/shared/memory_report.rs (ledger against
cudaMemGetInfo every 10 s and at ready).
"""
from __future__ import annotations

import contextlib
import dataclasses
import json
import os
import threading
import time
from typing import Callable, Iterator


def _tensors(obj, seen: set, depth: int = 0) -> Iterator:
    """Every torch tensor reachable from ``obj`` through dataclass fields, ``__dict__``, dicts, lists and tuples."""
    import torch
    if depth > 6 or obj is None or isinstance(obj, (str, bytes, int, float, bool)):
        return
    if isinstance(obj, torch.Tensor):
        yield obj
        return
    if id(obj) in seen:
        return
    seen.add(id(obj))
    if isinstance(obj, dict):
        vals = obj.values()
    elif isinstance(obj, (list, tuple, set)):
        vals = obj
    elif dataclasses.is_dataclass(obj) and not isinstance(obj, type):
        vals = (getattr(obj, f.name, None) for f in dataclasses.fields(obj))
    elif type(obj).__module__.startswith("cuteafd_b200") and (hasattr(obj, "__dict__") or hasattr(type(obj), "__slots__")):
        vals = list(vars(obj).values()) if hasattr(obj, "__dict__") else []
        vals += [getattr(obj, s, None) for s in getattr(type(obj), "__slots__", ())]
    else:
        return
    for v in vals:
        yield from _tensors(v, seen, depth + 1)


@dataclasses.dataclass
class Entry:
    kind: str
    owner: str
    device: str
    nbytes: int
    count: int = 1


class MemoryLedger:
    def __init__(self, probe: Callable[[str], tuple[int, int]] | None = None) -> None:
        """``probe(device) -> (free, total)``; default asks the CUDA driver and returns (0, 0) for host memory."""
        self.entries: dict[tuple[str, str, str], Entry] = {}
        self.lock = threading.Lock()
        self.probe = probe or self._cuda_probe
        self._storages: dict[tuple[str, int], tuple[str, str]] = {}     # storage -> (kind, owner) that counted it
        self._spool = None
        self._reporter: threading.Thread | None = None
        self._stop = threading.Event()
        self.failures: list[dict] = []

    # ---- tagging --------------------------------------------------------------------------
    def tag(self, kind: str, owner: str, nbytes: int, device: str = "cuda:0", count: int = 1) -> None:
        with self.lock:
            e = self.entries.get((kind, owner, device))
            if e is None:
                self.entries[(kind, owner, device)] = Entry(kind, owner, device, int(nbytes), count)
            else:
                e.nbytes += int(nbytes)
                e.count += count

    def tag_tensor(self, kind: str, owner: str, t) -> int:
        """Counts the tensor's whole storage once, however many views of it are tagged."""
        st = t.untyped_storage()
        key = (str(t.device), st.data_ptr())
        with self.lock:
            if key in self._storages or st.nbytes() == 0:
                return 0
            self._storages[key] = (kind, owner)
        self.tag(kind, owner, st.nbytes(), str(t.device))
        return st.nbytes()

    def tag_tree(self, kind: str, owner: str, obj) -> int:
        return sum(self.tag_tensor(kind, owner, t) for t in _tensors(obj, set()))

    def release(self, kind: str, owner: str, device: str | None = None) -> None:
        with self.lock:
            for key in [k for k in self.entries if k[0] == kind and k[1] == owner and device in (None, k[2])]:
                del self.entries[key]
            for st in [k for k, v in self._storages.items() if v == (kind, owner) and device in (None, k[0])]:
                del self._storages[st]

    # ---- queries --------------------------------------------------------------------------
    def total(self, device: str | None = None) -> int:
        with self.lock:
            return sum(e.nbytes for e in self.entries.values() if device in (None, e.device))

    @staticmethod
    def _cuda_probe(device: str) -> tuple[int, int]:
        if not device.startswith("cuda"):
            return 0, 0
        try:
            import torch
            if torch.cuda.is_available():
                return torch.cuda.mem_get_info(torch.device(device))
        except Exception:                                         # noqa: BLE001
            pass
        return 0, 0

    def reconcile(self) -> dict:
        """Per device: tracked bytes against what the driver says is in use; ``untracked`` is the difference (the
        allocator's cache, library workspaces, the CUDA context, other processes)."""
        with self.lock:
            devices = sorted({e.device for e in self.entries.values()})
        out = {}
        for d in devices:
            free, total = self.probe(d)
            tracked = self.total(d)
            used = total - free if total else None
            out[d] = {"tracked": tracked, "free": free, "total": total, "used": used,
                      "untracked": None if used is None else used - tracked}
        return out

    def report(self) -> dict:
        with self.lock:
            ents = sorted(self.entries.values(), key=lambda e: (e.device, -e.nbytes))
        by_kind: dict[str, int] = {}
        for e in ents:
            by_kind[e.kind] = by_kind.get(e.kind, 0) + e.nbytes
        return {"tracked_bytes": sum(e.nbytes for e in ents), "by_kind": by_kind, "devices": self.reconcile(),
                "entries": [dataclasses.asdict(e) for e in ents], "failures": self.failures[-8:]}

    def lines(self) -> list[str]:
        rep = self.report()
        out = [f"[memory] tracked {rep['tracked_bytes'] / 2**30:.2f} GiB: " +
               ", ".join(f"{k} {v / 2**30:.2f}" for k, v in sorted(rep["by_kind"].items(), key=lambda kv: -kv[1]))]
        for d, r in rep["devices"].items():
            if r["total"]:
                out.append(f"[memory] {d}: used {r['used'] / 2**30:.2f} of {r['total'] / 2**30:.2f} GiB, "
                           f"untracked {r['untracked'] / 2**30:.2f} GiB")
        return out

    # ---- failure spool and periodic report -----------------------------------------------------
    def open_spool(self, path: str) -> None:
        """Open the failure file now, while the process is healthy."""
        os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
        self._spool = open(path, "a", buffering=1)

    def dump_failure(self, what: str, error: str = "") -> dict:
        rec = {"time": time.time(), "what": what, "error": error[:400], "devices": self.reconcile(),
               "by_kind": self.report()["by_kind"]}
        self.failures.append(rec)
        if self._spool is not None:
            try:
                self._spool.write(json.dumps(rec) + "\n")
                self._spool.flush()
            except OSError:
                pass
        return rec

    @contextlib.contextmanager
    def guard(self, what: str):
        """Allocation failures inside the block are recorded with the ledger's state, then re-raised."""
        try:
            yield
        except MemoryError as e:
            self.dump_failure(what, str(e))
            raise
        except RuntimeError as e:
            if "out of memory" in str(e).lower():
                self.dump_failure(what, str(e))
            raise

    def start_reporter(self, period_s: float = 10.0, log=print) -> None:
        if self._reporter is not None:
            return

        def loop() -> None:
            while not self._stop.wait(period_s):
                for line in self.lines():
                    log(line)
        self._reporter = threading.Thread(target=loop, name="memory-report", daemon=True)
        self._reporter.start()

    def stop_reporter(self) -> None:
        self._stop.set()
        if self._reporter is not None:
            self._reporter.join(timeout=2)
            self._reporter = None
        self._stop = threading.Event()


LEDGER = MemoryLedger()
