"""Failure detection for the attention / expert rank group: a terminal health latch, peer states and a
host-side heartbeat over the process group's key-value store.

Rules (same as the reference's transport health latch, rust/crates/cuteafd-transport/src/lib.rs:14-30, and its
terminal peer states, rust/crates/cuteafd-daemon/src/shared/peer_split.rs:70-76):

* The first failure records its reason; the latch never clears.  Every later request is refused with that
  reason instead of being launched, so no kernel is started against a peer that is known to be gone.
* A rank leaves only between steps.  The others learn of it on the host - a missed heartbeat, an explicit
  ``leaving`` mark, or a device status word reporting a wait that ran out - before their next launch.
* Recovery is restart: there is no elastic re-sharding.

Nothing here touches a GPU: device waits are bounded inside the kernels and report through the status word,
which ``check_device`` folds into the latch.
"""
from __future__ import annotations

import enum
import threading
import time
from dataclasses import dataclass, field


class PeerState(enum.Enum):
    ACTIVE = "active"
    ABORTING = "aborting"      # failure seen, in-flight work is being drained
    DRAINED = "drained"        # nothing in flight any more; resources can be released
    RETAINED = "retained"      # drain failed: pages / slots stay quarantined until restart


class HealthError(RuntimeError):
    """Raised for every request after the latch tripped."""


@dataclass
class HealthLatch:
    reason: str | None = None
    failed_at: float | None = None
    state: PeerState = PeerState.ACTIVE
    _lock: threading.Lock = field(default_factory=threading.Lock, repr=False)

    def trip(self, reason: str) -> bool:
        """Record the first failure.  Returns True when this call was the first."""
        with self._lock:
            if self.reason is not None:
                return False
            self.reason, self.failed_at, self.state = reason, time.time(), PeerState.ABORTING
            return True

    @property
    def ok(self) -> bool:
        return self.reason is None

    def require(self) -> None:
        if self.reason is not None:
            raise HealthError(f"exchange unavailable: {self.reason}")

    def drained(self, success: bool = True) -> None:
        with self._lock:
            if self.state == PeerState.ABORTING:
                self.state = PeerState.DRAINED if success else PeerState.RETAINED

    def check_device(self, status: int, where: str = "") -> None:
        """Fold a device status word (0 = ok) into the latch."""
        if status:
            names = {1: "TMA data never arrived", 2: "no free stage", 3: "accumulator never completed", 4: "epilogue never finished",
                     5: "peer flag never raised", 6: "bad argument", 7: "softmax never finished", 8: "split-K ticket"}
            self.trip(f"bounded device wait ran out ({names.get(status, status)}){' in ' + where if where else ''}")


class Heartbeat:
    """Each rank publishes a counter under ``hb/<rank>`` in the store every ``period`` seconds from a daemon thread
    and marks ``leaving/<rank>`` when it shuts down in order.  ``check`` (called between steps) trips the latch when
    a peer announced its exit or its counter has not moved for ``timeout`` seconds."""

    def __init__(self, store, rank: int, world: int, latch: HealthLatch, period: float = 0.2, timeout: float = 2.0):
        self.store, self.rank, self.world, self.latch = store, rank, world, latch
        self.period, self.timeout = period, timeout
        self._stop = threading.Event()
        self._seen: dict[int, tuple[int, float]] = {}
        self._beat = 0
        self._thread = threading.Thread(target=self._run, daemon=True)

    def start(self) -> "Heartbeat":
        self._publish()
        self._thread.start()
        return self

    def _publish(self) -> None:
        self._beat += 1
        self.store.set(f"hb/{self.rank}", str(self._beat))

    def _run(self) -> None:
        while not self._stop.wait(self.period):
            try:
                self._publish()
            except Exception:
                return

    def leave(self) -> None:
        """Orderly exit between steps: tell the peers first, then stop beating."""
        try:
            self.store.set(f"leaving/{self.rank}", "1")
        finally:
            self._stop.set()

    def stop(self) -> None:
        self._stop.set()

    def check(self, now: float | None = None) -> None:
        now = time.time() if now is None else now
        for r in range(self.world):
            if r == self.rank:
                continue
            try:
                if self.store.check([f"leaving/{r}"]):
                    self.latch.trip(f"rank {r} left the group")
                    continue
                beat = int(self.store.get(f"hb/{r}")) if self.store.check([f"hb/{r}"]) else 0
            except Exception as e:                       # the store itself is gone: its host rank died
                self.latch.trip(f"heartbeat store unreachable: {type(e).__name__}")
                return
            last = self._seen.get(r)
            if last is None or beat != last[0]:
                self._seen[r] = (beat, now)
            elif now - last[1] > self.timeout:
                self.latch.trip(f"rank {r} missed heartbeats for {now - last[1]:.1f} s")
