"""KV admission that never deadlocks: leases, top-ups and a banker's-rule safety check.

A request is admitted with a lease of (prompt pages + one decode chunk); before it outgrows the
lease it asks for another chunk.  A top-up is granted only if, afterwards, the free pages still
let at least one active request run to its declared maximum (banker's rule), so some request can
always finish and release pages.  A request that cannot be topped up stalls; it is never
truncated.  Counterpart: rust/crates/cuteafd-engine/src/reserve.rs:1-50,
rust/crates/cuteafd-daemon/src/shared/kv_reserve.rs.
"""
from __future__ import annotations

from dataclasses import dataclass

from .paged import PAGE

DECODE_CHUNK_TOKENS = 16_384


def pages_for(tokens: int) -> int:
    return (tokens + PAGE - 1) // PAGE


@dataclass
class Lease:
    rid: int
    leased_pages: int        # pages this request may hold
    used_pages: int          # pages it holds now
    max_pages: int           # pages it would hold at its maximum length
    shared_pages: int = 0    # pages borrowed from the prefix cache (not charged)

    @property
    def remaining_need(self) -> int:
        return max(0, self.max_pages - self.leased_pages)


class KvReserve:
    def __init__(self, total_pages: int, decode_chunk_tokens: int = DECODE_CHUNK_TOKENS):
        self.total = total_pages
        self.chunk_pages = pages_for(decode_chunk_tokens)
        self.leases: dict[int, Lease] = {}

    @property
    def leased(self) -> int:
        return sum(l.leased_pages for l in self.leases.values())

    @property
    def unleased(self) -> int:
        return self.total - self.leased

    def _safe(self, unleased: int, leases: list[Lease]) -> bool:
        """Banker's rule: some ordering lets every request reach its maximum."""
        pending = sorted(leases, key=lambda l: l.remaining_need)
        free = unleased
        for l in pending:
            if l.remaining_need > free:
                return False
            free += l.leased_pages            # it finishes and returns everything it held
        return True

    def lease(self, rid: int, prompt_tokens: int, max_new_tokens: int, shared_pages: int = 0) -> Lease | None:
        """Admit or refuse (None = keep the request queued)."""
        prompt_pages = max(0, pages_for(prompt_tokens) - shared_pages)
        max_pages = max(0, pages_for(prompt_tokens + max_new_tokens) - shared_pages)
        want = min(max_pages, prompt_pages + self.chunk_pages)
        if want > self.unleased:
            return None
        cand = Lease(rid, want, 0, max_pages, shared_pages)
        if not self._safe(self.unleased - want, list(self.leases.values()) + [cand]):
            return None
        self.leases[rid] = cand
        return cand

    def top_up(self, rid: int) -> bool:
        """Another decode chunk for ``rid``; False = stall this request for now."""
        l = self.leases[rid]
        if l.leased_pages >= l.max_pages:
            return True
        add = min(self.chunk_pages, l.max_pages - l.leased_pages)
        if add > self.unleased:
            return False
        l.leased_pages += add
        if not self._safe(self.unleased, list(self.leases.values())):
            l.leased_pages -= add
            return False
        return True

    def needs_top_up(self, rid: int, next_len_tokens: int) -> bool:
        l = self.leases[rid]
        return pages_for(next_len_tokens) - l.shared_pages > l.leased_pages

    def note_used(self, rid: int, pages: int) -> None:
        self.leases[rid].used_pages = pages

    def release(self, rid: int) -> None:
        self.leases.pop(rid, None)
