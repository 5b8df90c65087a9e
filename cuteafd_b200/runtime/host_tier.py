"""Glue between the device prefix cache and the pinned-host tier.

Eviction side: ``PrefixCache(spill=tier.spill)`` hands every evicted snapshot (tokens, kind, device pages, positional
mark, retained next-token result) to ``HostCache.store`` before its pages go back to the pool.  Admission side: after
the device radix was walked, ``try_restore`` asks the host tier for a longer stored prefix, copies its pages into
freshly allocated device pages within a time budget, re-enters the snapshot into the device radix (so the next request
shares it by reference) and returns the sequence to continue from.  A restore that cannot complete in time, or for
which no pages can be had, is a miss, never a request error.

Counterpart: rust/crates/cuteafd-engine/src/prefix/cache.rs:1040 (``make_room`` spilling into the host store),
rust/crates/cuteafd-hostcache/src/cache.rs:378-669 (store / lookup / restore).
"""
from __future__ import annotations

from .hostcache import HostCache, HostSnapshot
from .paged import PAGE, OutOfPages, PagePool, Sequence, SequenceTable
from .prefix_cache import PrefixCache, Snapshot, chain_hashes


class HostTier:
    def __init__(self, prefix: PrefixCache, pool: PagePool, table: SequenceTable, host: HostCache,
                 budget_s: float = 0.05, min_gain_tokens: int = PAGE):
        self.prefix, self.pool, self.table, self.host = prefix, pool, table, host
        self.budget_s, self.min_gain = budget_s, min_gain_tokens
        prefix.spill = self.spill

    # ---- eviction -------------------------------------------------------------------------------------------
    def spill(self, snap: Snapshot, pages: list[int]) -> None:
        keys = chain_hashes(list(snap.tokens), self.prefix.salt + snap.media_key)
        self.host.store(snap.tokens, snap.kind, pages, keys, mark=snap.mark, after=snap.after)

    # ---- admission ------------------------------------------------------------------------------------------
    def try_restore(self, tokens: list[int], have: int) -> tuple[Sequence, int, HostSnapshot] | None:
        """A stored prefix at least ``min_gain_tokens`` longer than the ``have`` tokens the device tier matched:
        returns (sequence holding the restored pages, tokens reusable, the host snapshot), else None."""
        self.host.tick()
        hs = self.host.lookup(tokens)
        if hs is None or hs.length < have + self.min_gain:
            return None
        pages: list[int] = []
        try:
            for _ in range(len(hs.slots)):
                pages.append(self.pool.alloc())
        except OutOfPages:
            for p in pages:
                self.pool.release(p)
            self.prefix.stats.restore_failures += 1
            return None
        if not self.host.restore(hs, pages, self.budget_s):
            for p in pages:
                self.pool.release(p)
            self.prefix.stats.restore_failures += 1
            return None
        seq = self.table.new()
        seq.pages, seq.tokens, seq.kv_len = pages, list(hs.key), hs.length
        self.prefix.capture(seq, hs.kind, mark=hs.mark, after=hs.after)       # back in the device radix, shared by reference
        self.prefix.stats.restored += 1
        length = hs.length
        if length >= len(tokens):
            # the whole request is stored: like the device tier, reuse the full pages below its last token, so the
            # recomputed rows see the same chunk shape whichever tier served the prefix
            length = ((len(tokens) - 1) // PAGE) * PAGE
        if length < hs.length:
            seq.tokens, seq.kv_len = seq.tokens[:length], length
        return seq, length, hs

    def describe(self) -> dict:
        s = self.host.stats
        return {"stored": s.stored, "store_skipped": s.store_skipped, "lookups": s.lookups, "hits": s.hits,
                "restored": s.restored, "restore_timeouts": s.restore_timeouts, "evicted": s.evicted,
                "shared_pages": s.shared_pages, "snapshots": len(self.host.snaps), "free_slots": len(self.host.free)}
