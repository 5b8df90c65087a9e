"""Loop abort: end a response that has fallen into an exact repetition loop, like a ``max_tokens`` finish.

Two rules over the generated token ids, disjoint by period:

* **F (short cycles, period 1..256).**  ``streak[P]`` counts consecutive positions with ``t[i] == t[i - P]``; the rule
  fires when ``streak[P] >= max((copies - 1) * P, span)``.  With the defaults (8 copies, span 1024) a single repeated
  token aborts at 1025 tokens and a 400-token run of zeros in a table does not abort at all.
* **R (long blocks, period > 256).**  A 32-token shingle slides over the output; a position counts as seen when that
  exact shingle has already occurred ``copies - 1`` times and its previous occurrence lies more than 256 tokens back;
  the rule fires after ``run`` consecutive seen positions.  With the defaults (8 copies, run 512) a block of period P
  fires at ``7 P + 543`` tokens.

``run = 0`` turns rule R off, ``span = 0`` rule F; the guard costs nothing when both are off.  The shingle table stops
growing at 65 536 entries (a reply that long without a loop simply stops being watched for new shingles).

The scheduler feeds every emitted token; a hit finishes the request with ``finish_reason = "length"`` and
``usage.finish_detail = "repetition"`` and counts in ``loop_aborts``.

Counterpart: rust/crates/cuteafd-daemon/src/shared/repeat_guard.rs (rules R and F, the period gate) and
shared/loop_abort.rs (knobs ``--loop-abort-run``, ``--loop-abort-copies``, ``--loop-fast-span``, ``--loop-fast-copies``).
"""
from __future__ import annotations

from dataclasses import dataclass

import numpy as np

SHINGLE = 32
FAST_WINDOW = 256
MAX_ENTRIES = 65536


@dataclass(frozen=True)
class LoopAbortConfig:
    run: int = 512
    copies: int = 8
    fast_span: int = 1024
    fast_copies: int = 8

    @property
    def enabled(self) -> bool:
        return self.run > 0 or self.fast_span > 0

    def guard(self):
        """A detector for one request: the C++ twin when the runtime library is there, this module's otherwise."""
        if not self.enabled:
            return None
        try:
            from .native import NativeRepeatGuard
            return NativeRepeatGuard(self)
        except (OSError, AttributeError, ImportError):
            return RepeatGuard(self)


class RepeatGuard:
    def __init__(self, cfg: LoopAbortConfig = LoopAbortConfig()):
        self.cfg = cfg
        self.copies = max(2, min(64, cfg.copies))
        self.fast_copies = max(2, min(64, cfg.fast_copies))
        self.pushed = 0
        self.hit: dict | None = None
        # rule F: the last FAST_WINDOW tokens and one streak per period
        self._ring = np.full(FAST_WINDOW, -1, dtype=np.int64)
        self._streak = np.zeros(FAST_WINDOW + 1, dtype=np.int64)
        periods = np.arange(1, FAST_WINDOW + 1)
        self._need = np.maximum((self.fast_copies - 1) * periods, max(cfg.fast_span, 1))
        self._periods = periods
        # rule R: shingle -> [occurrences, index of the last one]
        self._tail: list[int] = []
        self._seen: dict[int, list[int]] = {}
        self._consecutive = 0

    def push(self, token: int) -> bool:
        """Feed one generated token; True once a rule has fired (and on every later call)."""
        if self.hit is not None:
            return True
        i = self.pushed
        self.pushed += 1
        if self.cfg.fast_span > 0:
            # token i - P sits at ring slot (i - P) mod FAST_WINDOW; slots never written hold -1
            prev = self._ring[(i - self._periods) % FAST_WINDOW]
            same = (prev == token) & (self._periods <= i)
            st = self._streak[1:]
            st[:] = np.where(same, st + 1, 0)
            fired = np.nonzero(st >= self._need)[0]
            self._ring[i % FAST_WINDOW] = token
            if fired.size:
                self.hit = {"rule": "fast", "period": int(fired[0]) + 1, "at": self.pushed}
                return True
        if self.cfg.run > 0:
            self._tail.append(token)
            if len(self._tail) > SHINGLE:
                del self._tail[0]
            if len(self._tail) == SHINGLE:
                key = hash(tuple(self._tail))
                rec = self._seen.get(key)
                if rec is None:
                    if len(self._seen) < MAX_ENTRIES:
                        self._seen[key] = [1, i]
                    self._consecutive = 0
                else:
                    period = i - rec[1]
                    seen = rec[0] >= self.copies - 1 and period > FAST_WINDOW
                    rec[0] = min(rec[0] + 1, 1 << 15)
                    rec[1] = i
                    self._consecutive = self._consecutive + 1 if seen else 0
                    if self._consecutive >= self.cfg.run:
                        self.hit = {"rule": "repeat", "period": period, "at": self.pushed}
                        return True
        return False
