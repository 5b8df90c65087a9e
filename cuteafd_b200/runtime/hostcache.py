"""Pinned-host tier of the prefix cache: write-behind store of evicted snapshots, exact page
sharing between stored snapshots, restores through an asynchronous copy engine, budgeted waits,
and a simulator that drives the store on a virtual clock.

The copy engine is a trait: ``CudaCopyEngine`` moves KV pages between the device pools and pinned
host buffers on dedicated streams; ``StubCopyEngine`` models bandwidth and latency on a virtual
clock so every policy decision is testable on CPU.  Counterpart:
rust/crates/cuteafd-hostcache/src/{lib.rs:1-77,cache.rs:126-669,snapshot.rs,pool.rs,copy.rs:1-40,
sim.rs:1-40}; quota rule rust/crates/cuteafd-core/src/prefix.rs:16-23 (min(32 GiB, 25% RAM),
snapshots under 512 tokens are not stored).
"""
from __future__ import annotations

import os
import random
from dataclasses import dataclass, field
from typing import Protocol

MIN_STORE_TOKENS = 512
GIB = 1 << 30


def default_quota_bytes() -> int:
    try:
        ram = os.sysconf("SC_PAGE_SIZE") * os.sysconf("SC_PHYS_PAGES")
    except (ValueError, OSError):
        ram = 64 * GIB
    return min(32 * GIB, ram // 4)


class CopyEngine(Protocol):
    def now(self) -> float: ...
    def store(self, device_pages: list[int], host_slots: list[int]) -> object: ...     # returns a ticket
    def restore(self, host_slots: list[int], device_pages: list[int]) -> object: ...
    def done(self, ticket: object) -> bool: ...
    def wait(self, ticket: object, budget_s: float) -> bool: ...


@dataclass
class _Ticket:
    finish: float
    nbytes: int


class StubCopyEngine:
    """Virtual-clock model: each direction is a queue with fixed latency and bandwidth."""

    def __init__(self, page_bytes: int, bandwidth_gbs: float = 50.0, latency_s: float = 20e-6):
        self.page_bytes, self.bw, self.lat = page_bytes, bandwidth_gbs * 1e9, latency_s
        self.clock = 0.0
        self.busy_until = {"store": 0.0, "restore": 0.0}
        self.copied = {"store": 0, "restore": 0}
        self.fail_next = False

    def now(self) -> float:
        return self.clock

    def advance(self, dt: float) -> None:
        self.clock += dt

    def _enqueue(self, kind: str, n_pages: int) -> _Ticket:
        nbytes = n_pages * self.page_bytes
        start = max(self.clock, self.busy_until[kind])
        fin = start + self.lat + nbytes / self.bw
        self.busy_until[kind] = fin
        self.copied[kind] += nbytes
        if self.fail_next:
            self.fail_next = False
            fin = float("inf")
        return _Ticket(fin, nbytes)

    def store(self, device_pages, host_slots):
        return self._enqueue("store", len(device_pages))

    def restore(self, host_slots, device_pages):
        return self._enqueue("restore", len(host_slots))

    def done(self, t: _Ticket) -> bool:
        return self.clock >= t.finish

    def wait(self, t: _Ticket, budget_s: float) -> bool:
        if t.finish - self.clock <= budget_s:
            self.clock = max(self.clock, t.finish)
            return True
        self.clock += budget_s
        return False


class CudaCopyEngine:
    """Device pages <-> pinned host slots on two side streams (one per direction)."""

    def __init__(self, kv_pools: list, host_slots: int):
        import torch
        self.torch = torch
        self.pools = kv_pools                                   # list of [num_pages, ...] device tensors
        self.host = [torch.empty((host_slots, *p.shape[1:]), dtype=p.dtype).pin_memory() for p in kv_pools]
        self.s_store, self.s_restore = torch.cuda.Stream(), torch.cuda.Stream()

    def now(self) -> float:
        import time
        return time.monotonic()

    def _copy(self, stream, pairs, to_host: bool):
        torch = self.torch
        stream.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(stream):
            for dev_page, slot in pairs:
                for pool, host in zip(self.pools, self.host):
                    if to_host:
                        host[slot].copy_(pool[dev_page], non_blocking=True)
                    else:
                        pool[dev_page].copy_(host[slot], non_blocking=True)
            ev = torch.cuda.Event()
            ev.record(stream)
        return ev

    def store(self, device_pages, host_slots):
        """The evicted pages go back to the pool as soon as this returns, so the compute stream is made to wait for the
        copy: nothing launched later can overwrite a page before its bytes have left."""
        ev = self._copy(self.s_store, list(zip(device_pages, host_slots)), True)
        self.torch.cuda.current_stream().wait_event(ev)
        return ev

    def restore(self, host_slots, device_pages):
        return self._copy(self.s_restore, list(zip(device_pages, host_slots)), False)

    def done(self, ev) -> bool:
        return ev.query()

    def wait(self, ev, budget_s: float) -> bool:
        import time
        t0 = time.monotonic()
        while not ev.query():
            if time.monotonic() - t0 > budget_s:
                return False
            time.sleep(20e-6)
        return True


@dataclass
class HostSnapshot:
    key: tuple[int, ...]                 # the token ids
    kind: str
    length: int
    slots: list[int]                     # host slot per page (shared slots are refcounted)
    chunk_keys: list[bytes]
    ticket: object = None                # pending store
    last_use: float = 0.0
    mark: object = None
    after: object = None


@dataclass
class HostStats:
    stored: int = 0
    store_skipped: int = 0
    lookups: int = 0
    hits: int = 0
    restored: int = 0
    restore_timeouts: int = 0
    evicted: int = 0
    shared_pages: int = 0


class HostCache:
    """Write-behind store keyed by token ids; pages with the same chained chunk hash share a slot."""

    def __init__(self, engine: CopyEngine, slots: int, page_tokens: int = 64):
        self.engine, self.page_tokens = engine, page_tokens
        self.free = list(range(slots - 1, -1, -1))
        self.slot_refs: dict[int, int] = {}
        self.by_chunk: dict[bytes, int] = {}          # chained chunk hash -> slot
        self.chunk_of: dict[int, bytes] = {}
        self.snaps: dict[tuple[int, ...], HostSnapshot] = {}
        self.stats = HostStats()

    # ---- store -------------------------------------------------------------------------------------
    def store(self, tokens: tuple[int, ...], kind: str, device_pages: list[int], chunk_keys: list[bytes],
              mark=None, after=None) -> bool:
        """Queue an evicted snapshot for the host tier (returns False when it is not worth keeping
        or there is no room even after eviction)."""
        if len(tokens) < MIN_STORE_TOKENS or tokens in self.snaps:
            self.stats.store_skipped += 1
            return False
        n = len(device_pages)
        keys = list(chunk_keys) + [None] * (n - len(chunk_keys))       # the partial tail has no shareable key
        def missing() -> int:
            return sum(1 for k in keys if k is None or k not in self.by_chunk)

        # evicting may drop pages this snapshot hoped to share: recount after every eviction
        while len(self.free) < missing() and self._evict_one():
            pass
        need = missing()
        if len(self.free) < need:
            self.stats.store_skipped += 1
            return False
        slots, copy_dev, copy_slot = [], [], []
        for page, k in zip(device_pages, keys):
            if k is not None and k in self.by_chunk:
                s = self.by_chunk[k]
                self.slot_refs[s] += 1
                self.stats.shared_pages += 1
            else:
                s = self.free.pop()
                self.slot_refs[s] = 1
                if k is not None:
                    self.by_chunk[k] = s
                    self.chunk_of[s] = k
                copy_dev.append(page)
                copy_slot.append(s)
            slots.append(s)
        ticket = self.engine.store(copy_dev, copy_slot) if copy_dev else None
        self.snaps[tokens] = HostSnapshot(tokens, kind, len(tokens), slots, [k for k in keys if k], ticket,
                                          self.engine.now(), mark, after)
        self.stats.stored += 1
        return True

    # ---- lookup / restore --------------------------------------------------------------------------
    def lookup(self, tokens: list[int]) -> HostSnapshot | None:
        """Longest stored snapshot that is a prefix of ``tokens``."""
        self.stats.lookups += 1
        best = None
        t = tuple(tokens)
        for key, s in self.snaps.items():
            if s.length <= len(t) and t[:s.length] == key and (best is None or s.length > best.length):
                best = s
        if best is not None:
            self.stats.hits += 1
            best.last_use = self.engine.now()
        return best

    def restore(self, snap: HostSnapshot, device_pages: list[int], budget_s: float = 0.05) -> bool:
        """Copy the snapshot's pages into freshly allocated device pages.  A pending store is
        waited for first; if either wait exceeds the budget the restore is abandoned (a miss)."""
        if snap.ticket is not None and not self.engine.done(snap.ticket):
            if not self.engine.wait(snap.ticket, budget_s):
                self.stats.restore_timeouts += 1
                return False
        t = self.engine.restore(snap.slots, device_pages)
        if not self.engine.wait(t, budget_s):
            self.stats.restore_timeouts += 1
            return False
        self.stats.restored += 1
        return True

    # ---- eviction ----------------------------------------------------------------------------------
    def _evict_one(self) -> bool:
        if not self.snaps:
            return False
        victim = min(self.snaps.values(), key=lambda s: (s.kind != "prompt", s.last_use))
        self.drop(victim.key)
        self.stats.evicted += 1
        return True

    def drop(self, key: tuple[int, ...]) -> None:
        s = self.snaps.pop(key, None)
        if s is None:
            return
        for slot in s.slots:
            self.slot_refs[slot] -= 1
            if self.slot_refs[slot] == 0:
                del self.slot_refs[slot]
                k = self.chunk_of.pop(slot, None)
                if k is not None:
                    self.by_chunk.pop(k, None)
                self.free.append(slot)

    def tick(self) -> int:
        """Retire finished stores; returns how many are still pending."""
        pending = 0
        for s in self.snaps.values():
            if s.ticket is not None:
                if self.engine.done(s.ticket):
                    s.ticket = None
                else:
                    pending += 1
        return pending

    def check_invariants(self) -> None:
        used = set(self.slot_refs)
        assert not (used & set(self.free)), "a slot is both free and referenced"
        counts: dict[int, int] = {}
        for s in self.snaps.values():
            for slot in s.slots:
                counts[slot] = counts.get(slot, 0) + 1
        assert counts == self.slot_refs, "slot refcounts drifted from the snapshots"
        for k, slot in self.by_chunk.items():
            assert self.chunk_of.get(slot) == k


def simulate(seed: int, steps: int = 400, slots: int = 64, page_bytes: int = 3 << 20) -> HostStats:
    """Seeded random interleaving of stores, lookups, restores, drops and clock advances with the
    invariants checked after every step (the reference's hostcache simulator, sim.rs)."""
    from .prefix_cache import chain_hashes
    rng = random.Random(seed)
    eng = StubCopyEngine(page_bytes)
    hc = HostCache(eng, slots)
    prefixes = [[rng.randrange(1000) for _ in range(640)] for _ in range(4)]
    known: list[tuple[int, ...]] = []
    for _ in range(steps):
        op = rng.random()
        if op < 0.4:
            base = rng.choice(prefixes)
            toks = tuple(base[: rng.choice((512, 576, 640))] + [rng.randrange(1000) for _ in range(rng.choice((0, 30, 64, 130)))])
            n_pages = (len(toks) + 63) // 64
            hc.store(toks, rng.choice(("prompt", "turn")), list(range(n_pages)), chain_hashes(list(toks)))
            known.append(toks)
        elif op < 0.7 and known:
            toks = list(rng.choice(known)) + [1, 2, 3]
            s = hc.lookup(toks)
            if s is not None:
                if rng.random() < 0.1:
                    eng.fail_next = True
                hc.restore(s, list(range(len(s.slots))), budget_s=rng.choice((1e-6, 1e-3, 1.0)))
        elif op < 0.8 and known:
            hc.drop(rng.choice(known))
        else:
            eng.advance(rng.choice((1e-5, 1e-3, 0.1)))
            hc.tick()
        hc.check_invariants()
    return hc.stats
