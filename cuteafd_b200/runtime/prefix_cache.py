"""Exact KV prefix cache, device tier: a radix index over raw token ids whose nodes hold
refcounted KV pages.

A *snapshot* is taken at prompt end and at turn end.  Its full pages enter the radix by reference
(no copy); a partial tail page is kept as a tail entry on the last node.  Admission walks the
radix with the new request's tokens: matched full pages are shared with the new sequence by
reference, a matched partial tail is copied on first write (copy-on-write), and the request
prefills only the unmatched suffix.  Bytes are never recomputed or converted, so a restored state
is the captured state bit for bit.  Two banks (prompt, turn) with LRU eviction, prompt snapshots
first; an evicted snapshot may spill to the pinned-host tier.  A restore that cannot complete is a
miss, never a request error.

Counterpart: rust/crates/cuteafd-engine/src/prefix/{mod.rs:1-35,cache.rs:1-140,357-1178,pages.rs,
entry.rs,chain.rs}, rust/crates/cuteafd-core/src/prefix.rs:1-140 (retention, radix).
"""
from __future__ import annotations

import hashlib
import struct
from dataclasses import dataclass, field
from typing import Callable

from .paged import PAGE, OutOfPages, PagePool, Sequence, SequenceTable

PROMPT, TURN = "prompt", "turn"
MIN_SNAPSHOT_TOKENS = 64


def chain_hashes(tokens: list[int], salt: bytes = b"") -> list[bytes]:
    """One hash per full 64-token chunk, each chained to the previous (cheap equality of prefixes)."""
    out, prev = [], hashlib.blake2b(salt, digest_size=16).digest()
    for i in range(0, len(tokens) - len(tokens) % PAGE, PAGE):
        h = hashlib.blake2b(prev + struct.pack(f"<{PAGE}i", *tokens[i:i + PAGE]), digest_size=16).digest()
        out.append(h)
        prev = h
    return out


@dataclass
class Node:
    key: bytes
    page: int
    parent: "Node | None"
    children: dict[bytes, "Node"] = field(default_factory=dict)
    refs: int = 0                                  # snapshots whose path passes through this node
    tails: dict[int, "Snapshot"] = field(default_factory=dict)   # snapshot id -> snapshot ending here with a partial page


@dataclass
class Snapshot:
    sid: int
    kind: str
    length: int
    tokens: tuple[int, ...]
    node: Node | None                 # last full-page node (None when shorter than a page)
    tail_page: int | None             # partial last page (retained), None when length % 64 == 0
    mark: object = None               # positional extras (drafter state, recurrent state ...)
    after: object = None              # next-token logits / token retained for whole hits
    last_use: int = 0
    media_key: bytes = b""

    @property
    def pages(self) -> int:
        return (self.length + PAGE - 1) // PAGE


@dataclass
class Match:
    length: int                       # tokens reusable
    pages: list[int]                  # pages to share, in order (the last may be a partial tail)
    tail_shared: bool                 # True when the last page is a shared partial tail (copy before writing)
    snapshot: Snapshot | None
    whole: bool = False               # the whole request was cached and ``after`` is available


@dataclass
class PrefixStats:
    lookups: int = 0
    hits: int = 0
    hit_tokens: int = 0
    lookup_tokens: int = 0
    captured: int = 0
    evicted: int = 0
    spilled: int = 0
    restored: int = 0
    restore_failures: int = 0


class PrefixCache:
    def __init__(self, pool: PagePool, table: SequenceTable, max_pages: int | None = None,
                 spill: Callable[[Snapshot, list[int]], None] | None = None, salt: bytes = b""):
        self.pool, self.table = pool, table
        self.root = Node(b"", 0, None)
        self.snapshots: dict[int, Snapshot] = {}
        self.max_pages = max_pages if max_pages is not None else pool.num_pages // 2
        self.max_entries = 0                      # retained snapshots at most (0 = bounded by pages alone); PREFIX_CACHE_ENTRIES
        self.held_pages = 0                       # pages retained by the cache (radix nodes + tails)
        self.clock = 0
        self.stats = PrefixStats()
        self.spill = spill
        self.salt = salt
        self._next = 1
        pool.on_exhausted = self.reclaim          # snapshots give pages back before an allocation fails

    # ---- lookup / admit ---------------------------------------------------------------------------
    def lookup(self, tokens: list[int], media_key: bytes = b"") -> Match:
        self.stats.lookups += 1
        self.stats.lookup_tokens += len(tokens)
        node, pages = self.root, []
        for h in chain_hashes(tokens, self.salt + media_key):
            nxt = node.children.get(h)
            if nxt is None:
                break
            node = nxt
            pages.append(node.page)
        length = len(pages) * PAGE
        best_tail: Snapshot | None = None
        rest = tokens[length:]
        for s in node.tails.values():
            t = s.length - length
            if 0 < t <= len(rest) and tuple(rest[:t]) == s.tokens[length:s.length] and (best_tail is None or s.length > best_tail.length):
                best_tail = s
        snap = None
        tail_shared = False
        if best_tail is not None:
            pages = pages + [best_tail.tail_page]
            length = best_tail.length
            tail_shared = True
            snap = best_tail
        whole = False
        if length >= len(tokens):
            # the entire request is cached: usable only when the next-token result was retained
            exact = next((s for s in self._ending_at(node, tokens) if s.after is not None), None)
            if exact is not None and exact.length == len(tokens):
                snap, whole = exact, True
            else:
                # leave at least one token to compute
                if tail_shared:
                    pages, tail_shared, snap = pages[:-1], False, None
                    length = len(pages) * PAGE
                if length >= len(tokens):
                    pages = pages[:-1]
                    length = len(pages) * PAGE
        if length:
            self.stats.hits += 1
            self.stats.hit_tokens += length
            self._touch(node if not whole else snap.node, snap)
        return Match(length, pages, tail_shared, snap, whole)

    def _ending_at(self, node: Node, tokens: list[int]):
        for s in self.snapshots.values():
            if s.length == len(tokens) and s.tokens == tuple(tokens):
                yield s

    def admit(self, tokens: list[int], media_key: bytes = b"") -> tuple[Sequence, Match]:
        """New sequence that shares the longest cached prefix; the caller prefills tokens[match.length:]."""
        m = self.lookup(tokens, media_key)
        seq = self.table.new()
        try:
            for p in m.pages:
                self.pool.retain(p)
            seq.pages = list(m.pages)
            seq.tokens = list(tokens[:m.length])
            seq.kv_len = m.length
        except Exception:
            self.stats.restore_failures += 1
            self.table.free(seq)
            seq = self.table.new()
            m = Match(0, [], False, None)
        return seq, m

    # ---- capture ----------------------------------------------------------------------------------
    def capture(self, seq: Sequence, kind: str = PROMPT, mark: object = None, after: object = None,
                media_key: bytes = b"") -> Snapshot | None:
        """Retain ``seq``'s KV up to its current length.  Pages are shared by reference."""
        length = seq.kv_len
        if length < MIN_SNAPSHOT_TOKENS:
            return None
        tokens = tuple(seq.tokens[:length])
        need = (length + PAGE - 1) // PAGE
        if not self.make_room(need):
            return None                           # larger than the cache's whole budget: not retained
        node = self.root
        hashes = chain_hashes(list(tokens), self.salt + media_key)
        path = []
        for i, h in enumerate(hashes):
            nxt = node.children.get(h)
            if nxt is None:
                nxt = Node(h, seq.pages[i], node)
                self.pool.retain(nxt.page)
                self.held_pages += 1
                node.children[h] = nxt
            node = nxt
            path.append(node)
        for n in path:
            n.refs += 1
        tail_page = None
        if length % PAGE:
            tail_page = seq.pages[len(hashes)]
            self.pool.retain(tail_page)
            self.held_pages += 1
        self.clock += 1
        s = Snapshot(self._next, kind, length, tokens, node if path else None, tail_page, mark, after, self.clock, media_key)
        self._next += 1
        self.snapshots[s.sid] = s
        if tail_page is not None:
            node.tails[s.sid] = s
        self.stats.captured += 1
        return s

    # ---- eviction ---------------------------------------------------------------------------------
    def _touch(self, node: Node | None, snap: Snapshot | None) -> None:
        self.clock += 1
        if snap is not None:
            snap.last_use = self.clock
        # snapshots whose path covers the matched node are kept warm too
        for s in self.snapshots.values():
            n = s.node
            while n is not None and n is not self.root:
                if n is node:
                    s.last_use = self.clock
                    break
                n = n.parent

    def release(self, sid: int, spill: bool = False) -> None:
        s = self.snapshots.pop(sid, None)
        if s is None:
            return
        if spill and self.spill is not None:
            pages = []
            n = s.node
            while n is not None and n is not self.root:
                pages.append(n.page)
                n = n.parent
            pages.reverse()
            if s.tail_page is not None:
                pages.append(s.tail_page)
            self.spill(s, pages)
            self.stats.spilled += 1
        if s.tail_page is not None:
            (s.node or self.root).tails.pop(s.sid, None)
            self.pool.release(s.tail_page)
            self.held_pages -= 1
        n = s.node
        while n is not None and n is not self.root:
            n.refs -= 1
            parent = n.parent
            if n.refs == 0 and not n.children and not n.tails:
                parent.children.pop(n.key, None)
                self.pool.release(n.page)
                self.held_pages -= 1
            n = parent
        self.stats.evicted += 1

    def make_room(self, pages_needed: int) -> bool:
        """Evict least-recently-used snapshots (prompt bank first) until the cache budget and the
        pool can take ``pages_needed`` more pages."""
        def victims():
            for kind in (PROMPT, TURN):
                for s in sorted((s for s in self.snapshots.values() if s.kind == kind), key=lambda s: s.last_use):
                    yield s
        while self.snapshots and (self.held_pages + pages_needed > self.max_pages
                                  or (self.max_entries and len(self.snapshots) >= self.max_entries)):
            v = next(victims(), None)
            if v is None:
                break
            self.release(v.sid, spill=True)
        return self.held_pages + pages_needed <= self.max_pages

    def reclaim(self, pages_needed: int) -> int:
        """Free pool pages for the allocator (admission pressure): least recently used snapshots go first, prompt
        bank before turn bank, spilling to the host tier when one is attached.  A snapshot whose pages are all shared
        with live sequences frees nothing; the walk continues.  Returns pages actually freed."""
        before = self.pool.free_pages
        order = sorted(self.snapshots.values(), key=lambda s: (s.kind != PROMPT, s.last_use))
        for v in order:
            if self.pool.free_pages - before >= pages_needed:
                break
            self.release(v.sid, spill=True)
        return self.pool.free_pages - before

    def clear(self) -> None:
        for sid in list(self.snapshots):
            self.release(sid)

    def describe(self) -> dict:
        st = self.stats
        return {"snapshots": len(self.snapshots), "held_pages": self.held_pages, "max_pages": self.max_pages,
                "prompt": sum(1 for s in self.snapshots.values() if s.kind == PROMPT),
                "turn": sum(1 for s in self.snapshots.values() if s.kind == TURN),
                "lookups": st.lookups, "hits": st.hits, "hit_tokens": st.hit_tokens, "lookup_tokens": st.lookup_tokens,
                "hit_rate": st.hit_tokens / st.lookup_tokens if st.lookup_tokens else 0.0,
                "captured": st.captured, "evicted": st.evicted, "spilled": st.spilled, "restored": st.restored,
                "restore_failures": st.restore_failures}
