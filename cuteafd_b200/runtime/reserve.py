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


def _split(first_page: int, pages: int, pools: int) -> list[int]:
    """How many of the logical pages [first_page, first_page + pages) land on each pool (page j lives on pool j mod n)."""
    out = [pages // pools] * pools
    for j in range(first_page + pages - pages % pools, first_page + pages):
        out[j % pools] += 1
    return out


class ParityReserve:
    """Leases over ``pools`` separate page pools with the pages of a sequence dealt round-robin (logical page j lives on
    pool j mod n): the layout of a context split, where every GPU of the group holds a share of every sequence's KV.
    A request is admitted, or topped up, only when every pool passes its own banker's rule; a refusal by one pool rolls
    the others back, so the pools never disagree about who holds a lease.

    Counterpart: the parity pools (two halves) of rust/crates/cuteafd-daemon/src/shared/kv_reserve.rs."""

    def __init__(self, pages_per_pool: int, pools: int = 2, decode_chunk_tokens: int = DECODE_CHUNK_TOKENS):
        self.pools = [KvReserve(pages_per_pool, decode_chunk_tokens) for _ in range(pools)]
        self.n = pools
        self.chunk_pages = pages_for(decode_chunk_tokens)
        self.meta: dict[int, dict] = {}          # rid -> {"shared", "leased", "max"} in logical pages

    @property
    def total(self) -> int:
        return sum(p.total for p in self.pools)

    @property
    def leased(self) -> int:
        return sum(p.leased for p in self.pools)

    def per_pool(self) -> list[dict]:
        return [{"total": p.total, "leased": p.leased} for p in self.pools]

    def _install(self, rid: int, shared: int, leased: int, max_pages: int) -> bool:
        """Set rid's lease to ``leased`` logical pages on every pool; all or nothing."""
        want = _split(shared, leased, self.n)
        most = _split(shared, max_pages, self.n)
        before = [p.leases.get(rid) for p in self.pools]
        done = []
        for p, w, m in zip(self.pools, want, most):
            old = p.leases.pop(rid, None)
            cand = Lease(rid, w, old.used_pages if old else 0, m, 0)
            if w > p.unleased or not p._safe(p.unleased - w, list(p.leases.values()) + [cand]):
                if old is not None:
                    p.leases[rid] = old
                for q, o in done:                                   # roll the earlier pools back
                    if o is None:
                        q.leases.pop(rid, None)
                    else:
                        q.leases[rid] = o
                return False
            p.leases[rid] = cand
            done.append((p, old))
        del before
        return True

    def lease(self, rid: int, prompt_tokens: int, max_new_tokens: int, shared_pages: int = 0) -> dict | None:
        prompt_pages = max(0, pages_for(prompt_tokens) - shared_pages)
        max_pages = max(0, pages_for(prompt_tokens + max_new_tokens) - shared_pages)
        want = min(max_pages, prompt_pages + self.chunk_pages)
        if not self._install(rid, shared_pages, want, max_pages):
            return None
        self.meta[rid] = {"shared": shared_pages, "leased": want, "max": max_pages}
        return self.meta[rid]

    def top_up(self, rid: int) -> bool:
        m = self.meta[rid]
        if m["leased"] >= m["max"]:
            return True
        more = min(m["max"], m["leased"] + self.chunk_pages)
        if not self._install(rid, m["shared"], more, m["max"]):
            return False
        m["leased"] = more
        return True

    def needs_top_up(self, rid: int, next_len_tokens: int) -> bool:
        m = self.meta[rid]
        return pages_for(next_len_tokens) - m["shared"] > m["leased"]

    def release(self, rid: int) -> None:
        self.meta.pop(rid, None)
        for p in self.pools:
            p.release(rid)
