"""Randomised interleavings of sequence and prefix-cache operations with the invariants checked after every step
(the reference tests its host cache the same way: a seeded interleaver with invariants after every step,
rust/crates/cuteafd-hostcache/src/sim.rs:1-40).

A model of the KV contents rides along: every "written" position stores its token in a page image, copy-on-write copies
the image, and after every operation each live sequence must read back exactly its own tokens through its page list.
Sharing by reference, tail copies, truncation, eviction under pressure and reclaim can therefore never hand a sequence
somebody else's rows without the test seeing it."""
import pytest
from hypothesis import HealthCheck, given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime.paged import PAGE, OutOfPages, PagePool, SequenceTable
from cuteafd_b200.runtime.prefix_cache import PROMPT, TURN, PrefixCache

STEMS = [[7] * 70, [7] * 64 + [9] * 80, [3, 4] * 100, [5] * 130]       # prompt families that share prefixes


def _pools():
    out = [PagePool]
    try:
        from cuteafd_b200.runtime.native import enabled
        from cuteafd_b200.runtime.paged import NativePagePool
        if enabled():
            out.append(NativePagePool)
    except Exception:                                                   # noqa: BLE001 - the library is optional on a CPU box
        pass
    return out


class World:
    def __init__(self, pool_cls, pages: int):
        self.pool = pool_cls(pages)
        self.table = SequenceTable(self.pool)
        self.cache = PrefixCache(self.pool, self.table, max_pages=pages // 2)
        self.image: dict[int, list] = {}            # page -> 64 cells of (token) or None
        self.live = []
        self.total = pages

    def _copy(self, src: int, dst: int) -> None:
        self.image[dst] = list(self.image.get(src, [None] * PAGE))

    def write(self, seq, tokens: list[int]) -> bool:
        start = seq.kv_len
        try:
            self.table.reserve(seq, start + len(tokens), copy_page=self._copy)
        except OutOfPages:
            return False
        for i, t in enumerate(tokens):
            p = seq.pages[(start + i) // PAGE]
            assert p != 0 and not self.pool.shared(p), "a write never lands in the zero page or in a page somebody else holds"
            self.image.setdefault(p, [None] * PAGE)[(start + i) % PAGE] = t
        seq.tokens.extend(tokens)
        seq.kv_len = start + len(tokens)
        return True

    def admit(self, prompt: list[int]) -> None:
        seq, m = self.cache.admit(prompt)
        assert m.length <= len(prompt) and seq.tokens == prompt[:m.length] and (m.whole or m.length < len(prompt))
        if not self.write(seq, prompt[m.length:]):
            self.table.free(seq)
            return
        self.live.append(seq)

    def check(self) -> None:
        holders: dict[int, int] = {}
        for s in self.live:
            assert len(s.pages) == (s.kv_len + PAGE - 1) // PAGE and s.tokens[:s.kv_len] == s.tokens
            for j, p in enumerate(s.pages):
                holders[p] = holders.get(p, 0) + 1
                n = min(PAGE, s.kv_len - j * PAGE)
                assert self.image[p][:n] == s.tokens[j * PAGE:j * PAGE + n], "a sequence reads back its own tokens"
        nodes, stack = 0, [self.cache.root]
        while stack:
            n = stack.pop()
            for c in n.children.values():
                holders[c.page] = holders.get(c.page, 0) + 1
                nodes += 1
                stack.append(c)
            for t in n.tails.values():
                holders[t.tail_page] = holders.get(t.tail_page, 0) + 1
                nodes += 1
        assert nodes == self.cache.held_pages <= self.cache.max_pages, "the cache counts what it holds and stays inside its budget"
        assert 0 not in holders
        assert self.pool.free_pages + len(holders) == self.total - 1, "every page is free or held, never both, never lost"
        for p, k in holders.items():
            assert self.pool.shared(p) == (k > 1)
        for s in self.cache.snapshots.values():                        # a snapshot's pages still hold its tokens
            pages, n = [], s.node
            while n is not None and n is not self.cache.root:
                pages.append(n.page)
                n = n.parent
            pages.reverse()
            if s.tail_page is not None:
                pages.append(s.tail_page)
            for j, p in enumerate(pages):
                k = min(PAGE, s.length - j * PAGE)
                assert tuple(self.image[p][:k]) == s.tokens[j * PAGE:j * PAGE + k]


OPS = st.lists(st.tuples(st.sampled_from(["admit", "extend", "truncate", "capture", "free", "reclaim"]),
                         st.integers(0, 3), st.integers(0, 200)), min_size=5, max_size=60)


@pytest.mark.parametrize("pool_cls", _pools())
@settings(max_examples=60, deadline=None, suppress_health_check=[HealthCheck.too_slow, HealthCheck.function_scoped_fixture])
@given(ops=OPS, pages=st.sampled_from([12, 24, 64]))
def test_interleaved_operations_keep_every_invariant(pool_cls, ops, pages):
    w = World(pool_cls, pages)
    for op, a, b in ops:
        if op == "admit":
            w.admit(STEMS[a] + [11 + b % 5] * (b % 90))
        elif w.live:
            s = w.live[b % len(w.live)]
            if op == "extend":
                w.write(s, [20 + a] * (1 + b % 70))
            elif op == "truncate" and s.kv_len > 1:
                w.table.truncate(s, max(1, s.kv_len - 1 - b % 5))
            elif op == "capture":
                w.cache.capture(s, PROMPT if a % 2 else TURN)
            elif op == "free":
                w.live.remove(s)
                w.table.free(s)
            elif op == "reclaim":
                w.cache.reclaim(1 + a)
        w.check()
    for s in list(w.live):
        w.table.free(s)
    w.live.clear()
    w.cache.clear()
    w.check()
    assert w.pool.free_pages == pages - 1
