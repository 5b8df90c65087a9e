"""Refcounted KV page pool and per-sequence page tables (64-token pages).

Pages are shared by reference between sequences and prefix-cache snapshots; a fork shares every
full page and copies only a partial tail (copy-on-write), as in the reference's ``RefPagePool``
(rust/crates/cuteafd-engine/src/prefix/pages.rs; rust/crates/cuteafd-core/src/kv_cache/allocator.rs).
Page 0 is reserved and stays zero.
"""
from __future__ import annotations

from dataclasses import dataclass, field

PAGE = 64


class OutOfPages(RuntimeError):
    pass


class PagePool:
    def __init__(self, num_pages: int):
        assert num_pages >= 2
        self.num_pages = num_pages
        self.refs = [0] * num_pages
        self.refs[0] = 1 << 30                       # reserved zero page
        self.free = list(range(num_pages - 1, 0, -1))
        # Called with the number of pages wanted when the free list is empty; whoever holds reclaimable pages (the
        # prefix cache's snapshots) gives some back.  The reference evicts snapshots under admission pressure the same
        # way (rust/crates/cuteafd-engine/src/prefix/cache.rs:1040, ``make_room``).
        self.on_exhausted = None

    @property
    def free_pages(self) -> int:
        return len(self.free)

    @property
    def usable_pages(self) -> int:
        """Pages that can ever hold KV (page 0 is reserved)."""
        return self.num_pages - 1

    def alloc(self) -> int:
        if not self.free and self.on_exhausted is not None:
            self.on_exhausted(8)                     # a few at a time: the next allocations are likely to follow
        if not self.free:
            raise OutOfPages("KV page pool exhausted")
        p = self.free.pop()
        self.refs[p] = 1
        return p

    def retain(self, p: int) -> None:
        assert self.refs[p] > 0
        self.refs[p] += 1

    def release(self, p: int) -> None:
        assert p != 0 and self.refs[p] > 0, p
        self.refs[p] -= 1
        if self.refs[p] == 0:
            self.free.append(p)

    def shared(self, p: int) -> bool:
        return self.refs[p] > 1


class NativePagePool(PagePool):
    """The same pool with its reference counts and free list in the C++ runtime (``csrc/rt/cafd_rt.cc``): what the
    serving backends construct when the library is present.  Same page order, same misuse checks."""

    def __init__(self, num_pages: int):
        from .native import NativePool
        assert num_pages >= 2
        self.num_pages = num_pages
        self._n = NativePool(num_pages)
        self.on_exhausted = None

    @property
    def free_pages(self) -> int:
        return self._n.free_pages

    def alloc(self) -> int:
        p = self._n.L.cafd_pool_alloc(self._n.h)
        if p < 0 and self.on_exhausted is not None:
            self.on_exhausted(8)
            p = self._n.L.cafd_pool_alloc(self._n.h)
        if p < 0:
            raise OutOfPages("KV page pool exhausted")
        return p

    def retain(self, p: int) -> None:
        assert self._n.L.cafd_pool_retain(self._n.h, p) == 0, p

    def release(self, p: int) -> None:
        assert self._n.L.cafd_pool_release(self._n.h, p) == 0, p

    def shared(self, p: int) -> bool:
        return self._n.refs(p) > 1


@dataclass
class Sequence:
    seq_id: int
    tokens: list[int] = field(default_factory=list)     # every token whose KV is (or will be) cached
    pages: list[int] = field(default_factory=list)
    kv_len: int = 0                                     # tokens whose KV is written

    def pages_needed(self, new_len: int) -> int:
        return max(0, (new_len + PAGE - 1) // PAGE - len(self.pages))


class SequenceTable:
    """Owns sequences and their pages; produces slot mappings for KV writes."""

    def __init__(self, pool: PagePool):
        self.pool = pool
        self.seqs: dict[int, Sequence] = {}
        self._next = 0

    def new(self) -> Sequence:
        s = Sequence(self._next)
        self._next += 1
        self.seqs[s.seq_id] = s
        return s

    def reserve(self, s: Sequence, new_len: int, copy_page=None) -> None:
        """Make room for ``new_len`` tokens.  A shared partial tail page is copied first
        (``copy_page(src, dst)`` performs the device copy)."""
        if s.pages and s.kv_len % PAGE and self.pool.shared(s.pages[-1]) and new_len > s.kv_len:
            fresh = self.pool.alloc()
            if copy_page is not None:
                copy_page(s.pages[-1], fresh)
            self.pool.release(s.pages[-1])
            s.pages[-1] = fresh
        for _ in range(s.pages_needed(new_len)):
            s.pages.append(self.pool.alloc())

    def slots(self, s: Sequence, start: int, n: int) -> list[int]:
        return [s.pages[(start + i) // PAGE] * PAGE + (start + i) % PAGE for i in range(n)]

    def fork(self, src: Sequence, length: int | None = None) -> Sequence:
        """New sequence sharing the first ``length`` tokens of ``src`` by reference."""
        length = src.kv_len if length is None else length
        s = self.new()
        n_pages = (length + PAGE - 1) // PAGE
        s.pages = list(src.pages[:n_pages])
        for p in s.pages:
            self.pool.retain(p)
        s.tokens, s.kv_len = list(src.tokens[:length]), length
        return s

    def truncate(self, s: Sequence, length: int) -> None:
        """Drop KV past ``length`` (rejected speculative rows)."""
        keep = (length + PAGE - 1) // PAGE
        for p in s.pages[keep:]:
            self.pool.release(p)
        del s.pages[keep:]
        s.kv_len = length
        del s.tokens[length:]

    def free(self, s: Sequence) -> None:
        for p in s.pages:
            self.pool.release(p)
        s.pages.clear()
        self.seqs.pop(s.seq_id, None)
