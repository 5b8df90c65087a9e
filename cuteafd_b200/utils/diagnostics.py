"""Diagnostics for a serving process: stack dumps on demand and on a stall, and the host heap monitor.

* ``install_stack_dump(path)``: SIGUSR1 writes the stack of every Python thread (named) to ``path`` (default stderr).
  The handler is registered through ``faulthandler`` as well, so a dump still comes out when the interpreter is stuck
  inside a native call that never returns to the bytecode loop.
* ``StallWatchdog``: the serve loop calls ``beat()`` every tick and ``busy(n)`` with the number of requests in flight;
  when there is work and no beat for ``limit_s`` seconds the watchdog writes one stack dump (once per stall) and counts
  it.  It never kills anything: the dump is the evidence, recovery is the operator's.
* ``HostHeapMonitor``: samples the process's resident set and the pinned-host bytes the caches report; warns once when
  the resident set passes a limit (a leak of pinned staging buffers shows up here long before the OOM killer).

Counterpart: rust/crates/cuteafd-daemon/src/shared/stack_dump.rs:1-40 (SIGUSR1 backtraces on stall), host heap
monitor and malloc tuning under rust/crates/cuteafd-daemon/src/shared/.
"""
from __future__ import annotations

import faulthandler
import os
import signal
import sys
import threading
import time
import traceback


def format_stacks() -> str:
    names = {t.ident: t.name for t in threading.enumerate()}
    out = [f"==== stack dump pid {os.getpid()} at {time.strftime('%Y-%m-%d %H:%M:%S')} ===="]
    for ident, frame in sys._current_frames().items():
        out.append(f"-- thread {names.get(ident, '?')} ({ident})")
        out.extend(l.rstrip("\n") for l in traceback.format_stack(frame))
    return "\n".join(out) + "\n"


def dump_stacks(path: str | None = None) -> str:
    text = format_stacks()
    if path:
        with open(path, "a") as f:
            f.write(text)
    else:
        sys.stderr.write(text)
    return text


_native_file = None


def install_stack_dump(path: str | None = None, signum: int = signal.SIGUSR1) -> bool:
    """Returns False where signals cannot be installed (not the main thread, or a platform without SIGUSR1)."""
    global _native_file
    try:
        signal.signal(signum, lambda *_: dump_stacks(path))
    except (ValueError, OSError, AttributeError):
        return False
    try:
        # second line of defence: faulthandler writes from C, without needing the interpreter loop; chain=True keeps
        # the Python-level handler above
        _native_file = open(path, "a") if path else sys.stderr
        faulthandler.register(signum, file=_native_file, all_threads=True, chain=True)
    except (ValueError, OSError, AttributeError, RuntimeError):
        pass
    return True


class StallWatchdog:
    def __init__(self, limit_s: float = 30.0, path: str | None = None, period_s: float | None = None, clock=time.monotonic):
        self.limit_s, self.path, self.clock = limit_s, path, clock
        self.period_s = period_s if period_s is not None else max(0.05, limit_s / 4)
        self._last = clock()
        self._busy = 0
        self._dumped = False
        self.stalls = 0
        self.last_dump = ""
        self._stop = threading.Event()
        self._thread: threading.Thread | None = None

    def beat(self) -> None:
        self._last = self.clock()
        self._dumped = False

    def busy(self, n: int) -> None:
        self._busy = n

    def check(self) -> bool:
        """One evaluation (the thread's body; tests call it with a fake clock).  True when a dump was written."""
        if self._busy > 0 and not self._dumped and self.clock() - self._last >= self.limit_s:
            self._dumped = True
            self.stalls += 1
            self.last_dump = dump_stacks(self.path) if self.path else format_stacks()
            return True
        return False

    def start(self) -> "StallWatchdog":
        def loop() -> None:
            while not self._stop.wait(self.period_s):
                self.check()
        self._thread = threading.Thread(target=loop, name="stall-watchdog", daemon=True)
        self._thread.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        if self._thread is not None:
            self._thread.join(timeout=2)


def resident_bytes() -> int:
    try:
        with open("/proc/self/statm") as f:
            return int(f.read().split()[1]) * os.sysconf("SC_PAGE_SIZE")
    except (OSError, ValueError, IndexError):
        return 0


class HostHeapMonitor:
    def __init__(self, limit_bytes: int = 0, pinned=None, read=resident_bytes, log=print):
        """``pinned``: optional callable returning the pinned-host bytes the caches hold."""
        self.limit, self.pinned, self.read, self.log = limit_bytes, pinned, read, log
        self.peak = 0
        self.warned = False

    def sample(self) -> dict:
        rss = self.read()
        self.peak = max(self.peak, rss)
        rec = {"resident_bytes": rss, "peak_bytes": self.peak, "pinned_bytes": self.pinned() if self.pinned else 0}
        if self.limit and rss > self.limit and not self.warned:
            self.warned = True
            self.log(f"[host-heap] resident {rss / 2**30:.2f} GiB passed the limit {self.limit / 2**30:.2f} GiB "
                     f"(pinned {rec['pinned_bytes'] / 2**30:.2f} GiB)")
        return rec
