"""C++ runtime structures against their Python models on identical random workloads."""
import random

import torch

from cuteafd_b200.runtime import native, sampling
from cuteafd_b200.runtime.paged import PagePool, SequenceTable
from cuteafd_b200.runtime.prefix_cache import PROMPT, TURN, PrefixCache
from cuteafd_b200.runtime.reserve import KvReserve


def test_native_page_pool_matches_python_pool_under_the_prefix_cache():
    """The C++ page pool behind the same ``SequenceTable`` + ``PrefixCache`` workload as the Python pool: every lookup,
    every page id and every free count agree, step by step (this is the pool the serving backends construct)."""
    from cuteafd_b200.runtime.paged import NativePagePool
    rng = random.Random(7)
    N = 96
    worlds = []
    for pool in (PagePool(N), NativePagePool(N)):
        tab = SequenceTable(pool)
        worlds.append((pool, tab, PrefixCache(pool, tab, max_pages=40)))
    bases = [[rng.randrange(500) for _ in range(300)] for _ in range(3)]
    live = [[], []]
    for step in range(300):
        base = rng.choice(bases)
        toks = base[: rng.choice((64, 100, 128, 200, 300))] + [rng.randrange(500) for _ in range(rng.choice((0, 5, 70)))]
        kind, drop = rng.choice((PROMPT, TURN)), rng.random() < 0.7
        seen = []
        for w, (pool, tab, cache) in enumerate(worlds):
            seq, m = cache.admit(toks)
            tab.reserve(seq, len(toks))
            seq.tokens, seq.kv_len = list(toks), len(toks)
            snap = cache.capture(seq, kind)
            live[w].append(seq)
            if drop or len(live[w]) > 3:
                tab.free(live[w].pop(0))
            seen.append((m.length, list(seq.pages), snap is not None, pool.free_pages, cache.held_pages))
        assert seen[0] == seen[1], (step, seen)
    assert worlds[1][2].held_pages > 0 and type(native.make_pool(8)).__name__ == "NativePagePool"
    import pytest
    with pytest.raises(AssertionError):
        worlds[1][0].release(0)                        # the reserved page is never released


def test_native_cow_fork_truncate():
    pool = native.NativePool(8)
    a = pool.new_seq()
    assert pool.reserve(a, 100)[0] == 2
    pool.set_len(a, 100)
    b = pool.fork(a)
    assert pool.pages(b) == pool.pages(a) and pool.refs(pool.pages(a)[1]) == 2
    added, cow = pool.reserve(b, 101)
    assert cow is not None and cow[0] == pool.pages(a)[1] and pool.pages(b)[1] == cow[1]
    assert pool.slots(a, 63, 2) == [pool.pages(a)[0] * 64 + 63, pool.pages(a)[1] * 64]
    pool.truncate(b, 64)
    assert len(pool.pages(b)) == 1
    pool.free(a); pool.free(b)
    assert pool.free_pages == 7
    c = pool.new_seq()
    assert pool.reserve(c, 8 * 64)[0] == -1


def test_reserve_matches_python_model():
    rng = random.Random(3)
    py, nat = KvReserve(200, 640), native.NativeReserve(200, 640)
    live = []
    for rid in range(1, 200):
        op = rng.random()
        if op < 0.5:
            p, m = rng.randrange(64, 3000), rng.randrange(64, 4000)
            a = py.lease(rid, p, m) is not None
            b = nat.lease(rid, p, m) is not None
            assert a == b
            if a:
                live.append(rid)
        elif op < 0.8 and live:
            r = rng.choice(live)
            n = rng.randrange(1, 8000)
            assert py.needs_top_up(r, n) == nat.needs_top_up(r, n)
            assert py.top_up(r) == nat.top_up(r)
        elif live:
            r = live.pop(rng.randrange(len(live)))
            py.release(r); nat.release(r)
        assert py.leased == nat.leased and py.unleased == nat.unleased and len(py.leases) == len(nat)
    assert type(native.make_reserve(10)).__name__ == "NativeReserve" and nat.total == 200


def test_native_sampler_matches_oracle():
    g = torch.Generator().manual_seed(0)
    for trial in range(40):
        logits = torch.randn(500, generator=g) * 3
        kw = dict(temperature=[0.0, 0.7, 1.3][trial % 3], top_p=[1.0, 0.9, 0.5][trial % 3], top_k=[None, 20, 3][(trial // 3) % 3],
                  min_p=[0.0, 0.05][trial % 2], seed=trial)
        P = sampling.SamplingParams(**kw)
        mask = (torch.rand(500, generator=g) > 0.3) if trial % 4 == 0 else None
        for pos in range(5):
            want = sampling.select_token(logits, P, pos, mask)
            got = native.sample_token(logits, position=pos, mask=mask, **kw)
            assert got == want, (trial, pos, kw)
        assert abs(native.sample_uniform(trial, 9) - P.uniform(9)) < 1e-7
    bad = torch.tensor([1.0, float("nan")])
    assert native.sample_token(bad) == -1
    assert native.sample_token(torch.ones(4), mask=torch.zeros(4, dtype=torch.bool)) == -2


def test_native_repeat_guard_matches_python():
    import random
    import time
    from cuteafd_b200.runtime.native import NativeRepeatGuard
    from cuteafd_b200.runtime.repeat_guard import LoopAbortConfig, RepeatGuard
    rnd = random.Random(4)
    streams = []
    for period in (1, 2, 7, 40, 255, 256, 257, 300, 700):
        head = [rnd.randrange(50000) for _ in range(rnd.randrange(0, 90))]
        blk = [rnd.randrange(50000) for _ in range(period)]
        streams.append(head + blk * (9000 // period + 2))
    streams.append([rnd.randrange(50000) for _ in range(6000)])                       # never fires
    streams.append([rnd.randrange(3) for _ in range(6000)])                            # tiny alphabet, no exact long loop
    for cfg in (LoopAbortConfig(), LoopAbortConfig(run=64, copies=3, fast_span=48, fast_copies=4), LoopAbortConfig(run=0),
                LoopAbortConfig(fast_span=0)):
        for toks in streams:
            a, b = RepeatGuard(cfg), NativeRepeatGuard(cfg)
            fa = next((i + 1 for i, t in enumerate(toks) if a.push(t)), None)
            fb = next((i + 1 for i, t in enumerate(toks) if b.push(t)), None)
            assert fa == fb, (cfg, fa, fb)
            assert (a.hit or {}).get("rule") == (b.hit or {}).get("rule") and (a.hit or {}).get("period") == (b.hit or {}).get("period")
    assert type(LoopAbortConfig().guard()).__name__ == "NativeRepeatGuard"
    g, t0 = NativeRepeatGuard(LoopAbortConfig()), time.perf_counter()
    for t in streams[-2]:
        g.push(t)
    assert (time.perf_counter() - t0) / 6000 < 20e-6


def test_native_wire_headers_match_python():
    import zlib
    from cuteafd_b200.parallel import wire
    from cuteafd_b200.runtime import native
    payload = bytes(range(256)) * 5 + b"tail"
    assert native.wire_crc32(payload) == zlib.crc32(payload) and native.wire_crc32(b"") == zlib.crc32(b"")
    req = wire.Request(wire.MOE, seq=9, flags=1, layer=4, rows=3, hidden=8, routes=5, dtype=wire.BF16, reply_dtype=wire.F32, unit=2,
                       plan=b"0123456789abcdef", payload=bytes(5 * 12 + 3 * 8 * 2))
    raw = req.pack()[:wire.HEADER]
    mine = native.wire_pack_request(wire.MOE, 1, 9, 4, 3, 8, 5, wire.BF16, wire.F32, 2, len(req.payload), zlib.crc32(req.payload), req.plan)
    assert mine == raw
    st, f = native.wire_parse_request(raw)
    assert st == wire.OK and (f["seq"], f["layer"], f["rows"], f["hidden"], f["routes"], f["unit"]) == (9, 4, 3, 8, 5, 2) and f["plan"] == req.plan
    for mutate, want in ((lambda b: b.__setitem__(0, 0x58), wire.BAD_MAGIC), (lambda b: b.__setitem__(8, 7), wire.BAD_VERSION),
                         (lambda b: b.__setitem__(28, 4), wire.BAD_SHAPE), (lambda b: b.__setitem__(40, 9), wire.BAD_DTYPE)):
        bad = bytearray(raw)
        mutate(bad)
        assert native.wire_parse_request(bytes(bad))[0] == want == wire.parse_request_header(bytes(bad))[3]
