"""Host-side runtime on CPU: page pool, prefix cache, KV leases, host tier, sampler oracle,
draft policy, and the scheduler over the oracle backend (lossless speculation, exact prefix
reuse, failure quarantine, admission limits)."""
import threading

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.ref.model import init_weights
from cuteafd_b200.runtime import hostcache, sampling, speculation
from cuteafd_b200.runtime.backends import OracleBackend
from cuteafd_b200.runtime.paged import PAGE, OutOfPages, PagePool, SequenceTable
from cuteafd_b200.runtime.prefix_cache import PROMPT, TURN, PrefixCache, chain_hashes
from cuteafd_b200.runtime.reserve import KvReserve
from cuteafd_b200.runtime.scheduler import FAIL_RETRY, FAIL_WORKER, Request, Scheduler, collect


# ---- pages ------------------------------------------------------------------------------------------
def test_page_pool_cow_and_truncate():
    pool = PagePool(8)
    tab = SequenceTable(pool)
    a = tab.new()
    tab.reserve(a, 100)
    a.kv_len, a.tokens = 100, list(range(100))
    assert len(a.pages) == 2 and 0 not in a.pages
    b = tab.fork(a)
    assert b.pages == a.pages and pool.shared(a.pages[1])
    copied = []
    tab.reserve(b, 101, copy_page=lambda s, d: copied.append((s, d)))
    assert copied and b.pages[1] != a.pages[1] and b.pages[0] == a.pages[0]
    tab.truncate(b, 64)
    assert len(b.pages) == 1
    tab.free(a); tab.free(b)
    assert pool.free_pages == 7
    with pytest.raises(OutOfPages):
        c = tab.new()
        tab.reserve(c, 8 * PAGE)


# ---- prefix cache ------------------------------------------------------------------------------------
def _seq_with(tab, tokens):
    s = tab.new()
    tab.reserve(s, len(tokens))
    s.tokens, s.kv_len = list(tokens), len(tokens)
    return s


def test_prefix_cache_share_tail_and_evict():
    pool = PagePool(64)
    tab = SequenceTable(pool)
    pc = PrefixCache(pool, tab, max_pages=12)
    base = list(range(200))
    s = _seq_with(tab, base)
    snap = pc.capture(s, PROMPT)
    assert snap.length == 200 and snap.tail_page == s.pages[3]
    # same prefix + new suffix: full pages and the partial tail are shared
    q, m = pc.admit(base + [7, 8, 9])
    assert m.length == 200 and m.tail_shared and q.pages == s.pages[:4]
    # a request equal to the cached prompt must still compute one token
    q2, m2 = pc.admit(base)
    assert 0 < m2.length < 200 and m2.length % PAGE == 0
    # diverging inside the second page: only the first page matches
    q3, m3 = pc.admit(base[:70] + [999] * 50)
    assert m3.length == 64
    for x in (q, q2, q3, s):
        tab.free(x)
    assert pc.held_pages == 4
    # budget: capturing more than max_pages evicts least recently used prompt snapshots first
    for i in range(4):
        t = _seq_with(tab, [1000 * (i + 1) + j for j in range(256)])
        pc.capture(t, TURN if i == 0 else PROMPT)
        tab.free(t)
    assert pc.held_pages <= 12 and pc.stats.evicted >= 1
    kinds = {s.kind for s in pc.snapshots.values()}
    assert TURN in kinds                                   # the turn snapshot outlives prompt snapshots
    pc.clear()
    assert pc.held_pages == 0 and pool.free_pages == 63


def test_chain_hash_is_prefix_stable():
    a = chain_hashes(list(range(200)))
    b = chain_hashes(list(range(128)) + [5] * 72)
    assert len(a) == 3 and a[:2] == b[:2] and a[2] != b[2]
    assert chain_hashes(list(range(200)), b"img") != a


# ---- reserve -----------------------------------------------------------------------------------------
def test_kv_reserve_bankers_rule():
    r = KvReserve(total_pages=100, decode_chunk_tokens=640)          # 10-page chunks
    a = r.lease(1, prompt_tokens=640, max_new_tokens=3200)           # 10 + 10 leased, max 60
    b = r.lease(2, prompt_tokens=640, max_new_tokens=3200)
    assert a and b and r.leased == 40
    assert r.lease(3, prompt_tokens=6400, max_new_tokens=64) is None  # would leave nobody able to finish
    assert r.top_up(1) and r.top_up(1)                               # 40 pages
    assert r.top_up(2)                                               # 30 pages -> 70 leased, 30 free
    assert r.top_up(1)                                               # 50: still safe (1 needs 10 more <= 20 free)
    assert not r.top_up(2) or r.unleased >= 0
    r.release(1)
    assert r.top_up(2)
    assert r.needs_top_up(2, 64 * 200) is True


# ---- host tier ----------------------------------------------------------------------------------------
def test_host_cache_sharing_timeouts_and_simulator():
    eng = hostcache.StubCopyEngine(page_bytes=1 << 20, bandwidth_gbs=1.0, latency_s=1e-3)
    hc = hostcache.HostCache(eng, slots=24)
    base = list(range(640))
    k = chain_hashes(base)
    assert hc.store(tuple(base), "prompt", list(range(10)), k)
    assert not hc.store(tuple(range(100)), "prompt", [1, 2], [])          # below the 512-token floor
    longer = base + list(range(64))
    assert hc.store(tuple(longer), "turn", list(range(11)), chain_hashes(longer))
    assert hc.stats.shared_pages == 10                                     # common pages stored once
    s = hc.lookup(longer + [1])
    assert s is not None and s.length == len(longer)
    assert not hc.restore(s, list(range(11)), budget_s=1e-6)               # store still in flight: miss
    eng.advance(1.0)
    assert hc.restore(s, list(range(11)), budget_s=1.0)
    hc.check_invariants()
    for seed in range(5):
        st = hostcache.simulate(seed, steps=300)
        assert st.stored > 0 and st.lookups > 0
    assert hostcache.default_quota_bytes() <= 32 << 30


# ---- sampling -----------------------------------------------------------------------------------------
def test_sampler_semantics():
    P = sampling.SamplingParams
    logits = torch.tensor([1.0, 3.0, 3.0, -2.0, 0.5])
    assert sampling.select_token(logits, P(), 0) == 1                       # greedy tie -> lowest id
    assert sampling.select_token(logits, P(temperature=1.0, top_k=1), 0) == 1
    mask = torch.tensor([True, False, False, True, True])
    assert sampling.select_token(logits, P(), 0, mask) == 0
    with pytest.raises(sampling.SamplingError):
        sampling.select_token(logits, P(), 0, torch.zeros(5, dtype=torch.bool))
    bad = logits.clone(); bad[3] = float("nan")
    toks, status = sampling.select_rows(torch.stack([logits, bad]), [P(), P()], [0, 0])
    assert toks[0] == 1 and status == [sampling.STATUS_OK, sampling.STATUS_NONFINITE]
    p = P(temperature=0.8, top_k=3, top_p=0.9, min_p=0.05, seed=42)
    draws = [sampling.select_token(logits, p, pos) for pos in range(200)]
    assert set(draws) <= {0, 1, 2} and len(set(draws)) > 1
    assert draws == [sampling.select_token(logits, p, pos) for pos in range(200)]     # pure in (seed, position)
    assert [p.uniform(i) for i in range(3)] != [P(temperature=0.8, seed=43).uniform(i) for i in range(3)]
    assert all(0.0 <= p.uniform(i) < 1.0 for i in range(1000))
    # top_p keeps the smallest prefix reaching the mass; uniform at both ends stays inside it
    sharp = torch.tensor([10.0, 0.0, 0.0, 0.0])
    assert sampling.select_token(sharp, P(temperature=1.0, top_p=0.5), 0, uniform=0.999) == 0
    assert sampling.accept_prefix([5, 6, 9, 1], [5, 6, 7]) == (2, 9)
    assert sampling.accept_prefix([5, 6, 7, 1], [5, 6, 7]) == (3, 1)
    with pytest.raises(sampling.SamplingError):
        P(temperature=3.0)


# ---- draft policy -------------------------------------------------------------------------------------
def test_history_policy_grows_and_shrinks():
    pol = speculation.DraftHistory(speculation.DrafterSpec(block=6))
    p = pol.plan(1, room=100)
    assert p.keep == 6                                           # cold neural rate 1.0: optimistic start
    for _ in range(12):                                          # everything rejected at position 0
        p = pol.plan(1, room=100)
        pol.observe(p, accepted=0)
    p = pol.plan(1, room=100)
    assert p.keep == 1 and p.explore == 0                        # only the explored position remains
    for _ in range(12):
        p = pol.plan(1, room=100)
        pol.observe(p, accepted=p.keep)
    assert pol.plan(1, room=100).keep >= 3                        # grows back
    assert pol.plan(1, room=2).keep <= 2                          # capped by room
    plans = [pol.plan(r, 100) for r in (10, 11, 12)]
    for q in plans:
        q.keep = 6
    pol.settle(plans, row_budget=9)
    assert sum(1 + q.keep + q.copy for q in plans) <= 9
    off = speculation.DraftHistory(speculation.DrafterSpec(block=6), control="off")
    assert off.plan(1, 100).keep == 0


def test_copy_continuation_needs_anchor():
    hist = [1, 2, 3, 4, 5, 6, 7, 8, 9, 10, 11, 12, 50, 1, 2, 3, 4, 5, 6]
    assert speculation.copy_continuation(hist, [7, 8, 9]) == [10, 11, 12, 50, 1, 2, 3, 4, 5, 6]
    assert speculation.copy_continuation(hist, [7, 8]) == []               # fewer than 3 agreeing drafts
    assert speculation.copy_continuation(hist, [7, 99, 9]) == []           # disagreement
    assert speculation.copy_continuation([1, 2, 3], [4, 5, 6]) == []


# ---- scheduler over the oracle --------------------------------------------------------------------------
@pytest.fixture(scope="module")
def oracle():
    cfg = tiny_moe()
    return cfg, init_weights(cfg, seed=0)


def _run(sched, reqs, steps=4000):
    for r in reqs:
        sched.submit(r)
    for _ in range(steps):
        if not sched.step() and sched.waiting.empty() and not sched.pending and not sched.prefilling and not sched.decoding:
            break
    return [collect(r, timeout=1.0) for r in reqs]


def test_scheduler_lossless_speculation_and_prefix_reuse(oracle):
    cfg, params = oracle
    g = torch.Generator().manual_seed(3)
    pattern = torch.randint(0, cfg.vocab_size, (12,), generator=g).tolist()
    prompt = (pattern * 9)[:100]                                  # repetitive: the n-gram drafter proposes
    plain = Scheduler(OracleBackend(cfg, params), drafter=None)
    base = _run(plain, [Request(prompt, max_tokens=24, record_rows=True, speculation=False)])[0]
    assert base["finish"] == "length" and len(base["tokens"]) == 24
    be = OracleBackend(cfg, params)
    spec = Scheduler(be, drafter=speculation.NgramDrafter(block=4))
    be_spec = spec.drafter
    be_spec.hist[1] = list(prompt)                                 # the drafter sees the prompt as history
    out = _run(spec, [Request(prompt, max_tokens=24, record_rows=True)])[0]
    assert out["tokens"] == base["tokens"]                         # ids identical with drafts on
    assert out["usage"]["speculation"]["cycles"] <= 24
    # the same prompt again: served from the prefix cache, identical tokens and row hashes
    again = _run(spec, [Request(prompt, max_tokens=24, record_rows=True, speculation=False)])[0]
    assert again["usage"]["cached_tokens"] >= 64
    assert again["tokens"] == base["tokens"]
    assert again["row_hashes"] == base["row_hashes"]
    assert be.prefix.stats.hits >= 1 and spec.snapshot()["finished"] == 2


def test_scheduler_batches_and_sampling_positions(oracle):
    cfg, params = oracle
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 70, 45)]
    P = sampling.SamplingParams(temperature=0.9, top_p=0.95, seed=11)
    solo = [_run(Scheduler(OracleBackend(cfg, params)), [Request(p, max_tokens=10, params=P)])[0]["tokens"] for p in prompts]
    together = _run(Scheduler(OracleBackend(cfg, params), max_active=3), [Request(p, max_tokens=10, params=P) for p in prompts])
    assert [o["tokens"] for o in together] == solo                 # batching does not change a sampled token


def test_scheduler_failure_quarantine_and_limits(oracle):
    cfg, params = oracle
    be = OracleBackend(cfg, params, fail_on_step=2)
    s = Scheduler(be, queue_depth=2)
    reqs = [Request([1, 2, 3, 4], max_tokens=8), Request([5, 6, 7], max_tokens=8), Request([9] * 5, max_tokens=8)]
    out = _run(s, reqs)
    assert out[2]["error"][0] == FAIL_RETRY                        # third request: queue full -> retry class
    assert all(o["error"] and o["error"][0] == FAIL_WORKER for o in out[:2])
    assert s.stats.failed == 2 and s.reserve.leased == 0
    assert s.stats.quarantined == 2 and len(be.quarantined) == 2   # a failed device step: pages kept out of the pool
    ok = _run(s, [Request([1, 2, 3], max_tokens=4)])[0]            # the scheduler keeps serving
    assert ok["finish"] == "length"
    bad = _run(s, [Request([], max_tokens=4)])[0]
    assert bad["error"][0] == "bad_request"
    # a request larger than the pool is refused with the retry class, not a crash
    tiny = Scheduler(OracleBackend(cfg, params, total_pages=4))
    big = _run(tiny, [Request([1] * 600, max_tokens=8)])[0]
    assert big["error"][0] == FAIL_RETRY


def test_prefix_cache_gives_pages_back_under_admission_pressure(oracle):
    """A warm cache never turns an admitted request into a failure: snapshots are evicted when the allocator runs
    dry, and a snapshot that exceeds the cache budget is not retained at all."""
    cfg, params = oracle
    be = OracleBackend(cfg, params, total_pages=16)
    s = Scheduler(be, max_active=1)
    g = torch.Generator().manual_seed(9)
    for _ in range(5):                                             # fills the cache's half of the pool with snapshots
        out = _run(s, [Request(torch.randint(0, cfg.vocab_size, (128,), generator=g).tolist(), max_tokens=2)])[0]
        assert out["finish"] == "length"
    held = be.prefix.held_pages
    assert held > 0 and held <= be.prefix.max_pages
    big = _run(s, [Request(torch.randint(0, cfg.vocab_size, (640,), generator=g).tolist(), max_tokens=2)])[0]
    assert big.get("error") is None and big["finish"] == "length"  # 10 pages + decode: needs the cache's pages
    assert be.prefix.stats.evicted >= 1 and s.stats.failed == 0
    assert be.prefix.held_pages <= be.prefix.max_pages
    assert s.reserve.total == 15                                   # the reserved zero page is not leasable


def test_host_tier_restores_an_evicted_snapshot_exactly(oracle):
    """Evicted snapshots go to the host tier; a later request for the same prompt is served from there with the same
    tokens and the same logit row hashes as when the device tier served it."""
    cfg, params = oracle
    be = OracleBackend(cfg, params, total_pages=40, host_slots=64)
    assert be.tier is not None and be.prefix.spill is not None
    s = Scheduler(be, max_active=1)
    g = torch.Generator().manual_seed(21)
    prompt = torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist()             # >= 512 tokens: worth storing
    cold = _run(s, [Request(prompt, max_tokens=6, record_rows=True, speculation=False)])[0]
    first = _run(s, [Request(prompt, max_tokens=6, record_rows=True, speculation=False)])[0]   # from the device tier
    assert first["usage"]["cached_tokens"] >= 512 and first["tokens"] == cold["tokens"]
    for _ in range(4):                                                                   # other traffic evicts it
        _run(s, [Request(torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist(), max_tokens=2)])
    assert be.prefix.stats.spilled >= 1 and be.tier.host.stats.stored >= 1
    assert not any(sn.tokens[:600] == tuple(prompt) for sn in be.prefix.snapshots.values())
    again = _run(s, [Request(prompt, max_tokens=6, record_rows=True, speculation=False)])[0]
    assert be.prefix.stats.restored >= 1 and be.tier.host.stats.restored >= 1
    assert again["usage"]["cached_tokens"] >= 512
    assert again["tokens"] == first["tokens"] and again["row_hashes"] == first["row_hashes"]
    be.tier.host.check_invariants()


def test_scheduler_thread_and_cancel(oracle):
    cfg, params = oracle
    s = Scheduler(OracleBackend(cfg, params))
    t = threading.Thread(target=s.run_forever, daemon=True)
    t.start()
    r1 = s.submit(Request([3, 4, 5, 6], max_tokens=6, stop_ids=()))
    r2 = s.submit(Request([3, 4, 5, 6], max_tokens=200))
    r2.cancelled.set()
    o1 = collect(r1, timeout=30)
    s.stop(); t.join(timeout=5)
    assert o1["finish"] == "length" and len(o1["tokens"]) == 6


def test_mtp_drafter_is_lossless_and_feeds_the_next_step():
    """Native MTP drafts: the depth runs on every verify step's rows, its draft for the bonus row is offered to the
    drafter, the next step verifies it; emitted tokens equal the run without speculation."""
    from cuteafd_b200.config import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    cfg = tiny_moe().replace(mtp_layers=1)
    params = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(9)
    prompt = torch.randint(0, cfg.vocab_size, (70,), generator=g).tolist()
    base = _run(Scheduler(OracleBackend(cfg.replace(mtp_layers=0), params), drafter=None),
                [Request(prompt, max_tokens=20, speculation=False)])[0]
    be = OracleBackend(cfg, params)
    assert be.has_mtp
    drafter = speculation.MtpDrafter()
    out = _run(Scheduler(be, drafter=drafter), [Request(prompt, max_tokens=20)])[0]
    assert out["tokens"] == base["tokens"]
    sp = out["usage"]["speculation"]
    assert drafter.offered >= 10 and sp["proposed"] >= 5 and sp["cycles"] <= 20


def test_two_decode_lanes_serve_alternately_without_changing_tokens(oracle):
    cfg, params = oracle
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (20, 33, 41, 27)]
    one = _run(Scheduler(OracleBackend(cfg, params), max_active=4), [Request(p, max_tokens=8) for p in prompts])
    sch = Scheduler(OracleBackend(cfg, params), max_active=4, decode_lanes=2)
    two = _run(sch, [Request(p, max_tokens=8) for p in prompts])
    assert [o["tokens"] for o in two] == [o["tokens"] for o in one]
    assert sch.stats.lane_rounds.get(0, 0) > 0 and sch.stats.lane_rounds.get(1, 0) > 0


def test_agentic_prefix_workload_on_the_oracle():
    """Shared prefix, several sessions and turns: most prompt tokens come from the cache, a turn served again from
    the warm cache reproduces its logit rows exactly, and a cold recompute emits the same tokens."""
    from cuteafd_b200.bench.agentic import run
    from cuteafd_b200.config import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)
    out = run(lambda: OracleBackend(cfg, params, total_pages=256, prefill_chunk=64, max_decode_rows=3), cfg.vocab_size,
              sessions=3, prefix=192, turns=3, append=24, decode=6, verify=3, concurrency=3)
    assert out["cache_share"] > 0.5 and out["restore_mismatches"] == 0 and out["cold_token_mismatches"] == 0
    assert out["emitted_tokens"] == 3 * 3 * 6


def test_prompt_packing_matches_one_at_a_time():
    """Short prompts that wait together share prefill steps; the generated tokens are those of serving them alone."""
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)
    g = torch.Generator().manual_seed(9)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (9, 21, 5, 40, 13)]

    def serve(max_active):
        sched = Scheduler(OracleBackend(cfg, params, prefill_chunk=64), max_active=max_active)
        reqs = [Request(prompt=list(p), max_tokens=5, speculation=False) for p in prompts]
        for r in reqs:
            sched.submit(r)
        out = [[] for _ in reqs]
        for _ in range(500):
            sched.step()
            for i, r in enumerate(reqs):
                while not r.events.empty():
                    ev = r.events.get()
                    if ev[0] == "tokens":
                        out[i] += ev[1]
            if sched.stats.finished == len(reqs):
                break
        assert sched.stats.finished == len(reqs)
        return out, sched.stats.packed_steps
    alone, p1 = serve(1)
    packed, p5 = serve(5)
    assert alone == packed and p1 == 0 and p5 >= 1


def test_repeat_guard_rules():
    """Rule F (short cycles) and rule R (long blocks) fire where their definitions say, and not on ordinary text."""
    import random
    from cuteafd_b200.runtime.repeat_guard import LoopAbortConfig, RepeatGuard
    rnd = random.Random(0)

    def fires_at(tokens_of, cfg=LoopAbortConfig()):
        g, i = RepeatGuard(cfg), 0
        while not g.push(tokens_of(i)):
            i += 1
            assert i < 100000
        return g.pushed, g.hit
    assert fires_at(lambda i: 7) == (1025, {"rule": "fast", "period": 1, "at": 1025})
    blk = [rnd.randrange(50000) for _ in range(40)]
    assert fires_at(lambda i: blk[i % 40])[0] == 40 + 1024
    big = [rnd.randrange(50000) for _ in range(300)]
    n, hit = fires_at(lambda i: big[i % 300])
    assert n == 7 * 300 + 543 and hit["rule"] == "repeat" and hit["period"] == 300
    # each rule has its own off switch
    n, hit = fires_at(lambda i: big[i % 300], LoopAbortConfig(run=64, copies=3, fast_span=0))
    assert hit["rule"] == "repeat" and n == 2 * 300 + 31 + 64
    g = RepeatGuard(LoopAbortConfig(run=0, fast_span=1024))
    assert not any(g.push(big[i % 300]) for i in range(5000))
    assert LoopAbortConfig(run=0, fast_span=0).guard() is None
    # ordinary text, and a 400-token run of one value inside it, pass
    g = RepeatGuard()
    text = [rnd.randrange(1, 50000) for _ in range(3000)]
    assert not any(g.push(t) for t in text[:1500] + [0] * 400 + text[1500:])


def test_scheduler_ends_a_looping_reply(oracle):
    from cuteafd_b200.runtime.repeat_guard import LoopAbortConfig
    cfg, params = oracle

    class OnlyToken:                       # a constraint that leaves one token: the reply is a period-1 loop
        def mask(self):
            m = torch.zeros(cfg.vocab_size, dtype=torch.bool)
            m[5] = True
            return m

        def advance(self, tok): pass
        def finished(self): return False

    sched = Scheduler(OracleBackend(cfg, params), loop_abort=LoopAbortConfig(run=0, fast_span=24, fast_copies=4))
    out = _run(sched, [Request([1, 2, 3], max_tokens=200, constraint=OnlyToken())])[0]
    assert out["finish"] == "length" and len(out["tokens"]) == 25 and set(out["tokens"]) == {5}
    assert out["usage"]["finish_detail"] == "repetition" and sched.snapshot()["loop_aborts"] == 1
    # with the detector off the same request runs to max_tokens
    off = _run(Scheduler(OracleBackend(cfg, params)), [Request([1, 2, 3], max_tokens=40, constraint=OnlyToken())])[0]
    assert len(off["tokens"]) == 40 and "finish_detail" not in off["usage"]


def test_speculation_trace_and_watchdog_hooks(oracle, tmp_path):
    import json
    from cuteafd_b200.utils.diagnostics import StallWatchdog
    from cuteafd_b200.utils.trace import JsonlTrace
    cfg, params = oracle
    sched = Scheduler(OracleBackend(cfg, params), drafter=speculation.NgramDrafter(block=4))
    path = str(tmp_path / "rounds.jsonl")
    sched.trace = JsonlTrace(path)
    sched.watchdog = StallWatchdog(limit_s=1000.0)
    pattern = [3, 9, 4, 7, 1, 8]
    out = _run(sched, [Request((pattern * 12)[:64], max_tokens=12)])[0]
    sched.trace.close()
    recs = [json.loads(l) for l in open(path)]
    assert len(recs) == sched.stats.decode_rounds and sched.trace.dropped == 0
    assert sum(sum(r["accepted"]) + len(r["accepted"]) for r in recs) >= len(out["tokens"]) - 1   # the first token came from prefill
    assert all({"round", "requests", "rows", "proposed", "accepted", "kept", "copied", "ts"} <= set(r) for r in recs)
    assert sched.watchdog.stalls == 0 and sched.watchdog._busy == 0        # the last step saw an empty engine


def test_parity_reserve_deals_pages_and_stays_consistent():
    from cuteafd_b200.runtime.reserve import ParityReserve, _split
    assert _split(0, 5, 2) == [3, 2] and _split(1, 5, 2) == [2, 3] and _split(3, 4, 2) == [2, 2] and _split(2, 7, 3) == [2, 2, 3]
    assert all(sum(_split(f, n, k)) == n for f in range(5) for n in range(12) for k in (1, 2, 3, 4))
    r = ParityReserve(pages_per_pool=10, pools=2, decode_chunk_tokens=128)           # chunk = 2 pages
    a = r.lease(1, prompt_tokens=64 * 5, max_new_tokens=64 * 4)                      # 5 prompt pages + 2: pools get 4 and 3
    assert a == {"shared": 0, "leased": 7, "max": 9} and [p["leased"] for p in r.per_pool()] == [4, 3]
    b = r.lease(2, prompt_tokens=64 * 3, max_new_tokens=64 * 2, shared_pages=1)      # logical pages 1..4: two on each pool
    assert b["leased"] == 4 and [p["leased"] for p in r.per_pool()] == [6, 5]
    # a request that would fit the sum of the pools but not one of them is refused, and nothing is left behind
    assert r.lease(3, prompt_tokens=64 * 9, max_new_tokens=64) is None
    assert [p["leased"] for p in r.per_pool()] == [6, 5] and all(3 not in p.leases for p in r.pools)
    assert r.needs_top_up(1, 64 * 7 + 1) and r.top_up(1) and r.meta[1]["leased"] == 9
    assert [p["leased"] for p in r.per_pool()] == [7, 6] and r.top_up(1)              # at the maximum: nothing more to take
    r.release(1)
    assert [p["leased"] for p in r.per_pool()] == [2, 2] and r.leased == 4 and r.total == 20
    # one pool is plain KvReserve
    one, plain = ParityReserve(20, pools=1, decode_chunk_tokens=128), KvReserve(20, 128)
    for rid, (p, m) in enumerate([(300, 200), (700, 64), (64, 2000)]):
        assert (one.lease(rid, p, m) is None) == (plain.lease(rid, p, m) is None)
    assert one.leased == plain.leased


def test_model_drafter_is_lossless_and_a_perfect_draft_model_is_fully_accepted(oracle):
    cfg, params = oracle
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, cfg.vocab_size, (48,), generator=g).tolist()
    base = _run(Scheduler(OracleBackend(cfg, params)), [Request(prompt, max_tokens=20, speculation=False)])[0]
    # the target itself as the draft model: every draft is what the target will pick
    perfect = speculation.ModelDrafter.from_oracle(cfg, params, block=4)
    s1 = Scheduler(OracleBackend(cfg, params), drafter=perfect)
    out = _run(s1, [Request(prompt, max_tokens=20)])[0]
    sp = out["usage"]["speculation"]
    assert out["tokens"] == base["tokens"] and sp["proposed"] > 0 and sp["accepted"] == sp["proposed"]
    assert sp["cycles"] < 20 and perfect.state == {}                       # fewer target steps than tokens; state dropped at finish
    # an unrelated draft model: drafts are mostly wrong, the reply is still the target's
    other = speculation.ModelDrafter.from_oracle(cfg, init_weights(cfg, seed=99), block=3)
    s2 = Scheduler(OracleBackend(cfg, params), drafter=other, draft_control="always") if "draft_control" in Scheduler.__init__.__code__.co_varnames else None
    out2 = _run(s2, [Request(prompt, max_tokens=20), Request(prompt[:30], max_tokens=12)])
    solo = _run(Scheduler(OracleBackend(cfg, params)), [Request(prompt[:30], max_tokens=12, speculation=False)])[0]
    assert out2[0]["tokens"] == base["tokens"] and out2[1]["tokens"] == solo["tokens"] and other.drafted > 0
    # the n-gram drafter now starts from the prompt and forgets finished requests
    ng = speculation.NgramDrafter(block=4)
    pattern = [5, 9, 2, 7, 3, 8] * 10
    s3 = Scheduler(OracleBackend(cfg, params), drafter=ng)
    _run(s3, [Request(pattern, max_tokens=8)])
    assert ng.hist == {}
    ng.begin(7, [1, 2, 3, 4, 1, 2, 3], 4)
    assert ng.draft(7, None, 4, 3)[0] == [1, 2, 3]


def test_profile_modes(oracle, tmp_path):
    import json
    from cuteafd_b200.utils.profile import Profile, parse_modes
    cfg, params = oracle
    with pytest.raises(ValueError):
        parse_modes("draft-timing,nsys")
    sched = Scheduler(OracleBackend(cfg, params), drafter=speculation.NgramDrafter(block=3))
    prof = Profile(parse_modes("draft-timing, expert-routes,census,step-timing"), str(tmp_path / "p"), period=2).attach(sched)
    out = _run(sched, [Request(([3, 1, 4, 1, 5, 9] * 8)[:40], max_tokens=10)])[0]
    assert len(out["tokens"]) == 10
    rep = prof.report()
    assert rep["draft"]["draft"]["calls"] >= 1 and rep["draft"]["begin"]["calls"] == 1 and 0 <= rep["draft"]["share_of_decode"] < 1
    assert rep["steps"]["decode"]["count"] == sched.stats.decode_rounds and rep["steps"]["prefill"]["count"] >= 1
    routes = [json.loads(l) for l in open(tmp_path / "p" / "expert_routes.jsonl")]
    census = [json.loads(l) for l in open(tmp_path / "p" / "census.jsonl")]
    assert routes and routes[-1]["usage"]["layers"] and census and census[-1]["verify_row_hist"]
    assert len(routes) == len(census) <= sched.stats.decode_rounds // 2 + 1


def test_usage_counts_the_round_that_ends_the_reply(oracle):
    cfg, params = oracle
    out = _run(Scheduler(OracleBackend(cfg, params)), [Request(list(range(1, 30)), max_tokens=5, speculation=False)])[0]
    assert len(out["tokens"]) == 5 and out["usage"]["speculation"]["cycles"] == 4      # one token from prefill, four decode rounds


def test_request_longer_than_the_context_is_refused_at_the_door():
    """A prompt + max_tokens beyond what one page-table row can describe is a client error at submit, not a failed step."""
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import FAIL_BAD_REQUEST, Request, Scheduler, collect
    cfg = tiny_moe()
    be = OracleBackend(cfg, init_weights(cfg, seed=0), total_pages=32)
    be.max_context_tokens = 256
    sched = Scheduler(be, max_active=2)
    r = sched.submit(Request(prompt=[1] * 250, max_tokens=16))
    out = collect(r, timeout=1)
    assert out["error"] and out["error"][0] == FAIL_BAD_REQUEST and "context" in out["error"][1]
    ok = sched.submit(Request(prompt=[1] * 200, max_tokens=16))
    for _ in range(200):
        sched.step()
    assert collect(ok, timeout=5)["error"] is None and sched.stats.rejected == 1


def test_block_drafter_drafts_a_block_in_one_pass_and_is_lossless(oracle):
    """The block drafter runs the draft model once per round over [last token, mask, mask, ...]; with the target itself
    as draft model its first position is always right (the others come from mask inputs), and whatever it proposes the
    reply is the target's."""
    cfg, params = oracle
    g = torch.Generator().manual_seed(12)
    prompt = torch.randint(0, cfg.vocab_size, (48,), generator=g).tolist()
    base = _run(Scheduler(OracleBackend(cfg, params)), [Request(prompt, max_tokens=20, speculation=False)])[0]
    blk = speculation.ModelDrafter.from_oracle(cfg, params, block=4, parallel=True)
    assert type(blk).__name__ == "BlockModelDrafter" and blk.mask_token == cfg.vocab_size - 1
    out = _run(Scheduler(OracleBackend(cfg, params), drafter=blk, draft_control="always"), [Request(prompt, max_tokens=20)])[0]
    sp = out["usage"]["speculation"]
    assert out["tokens"] == base["tokens"] and sp["proposed"] > 0 and sp["accepted"] >= sp["cycles"] - 2      # position 1 of every block
    assert blk.passes <= sp["cycles"] and blk.drafted >= 2 * blk.passes and blk.state == {}                    # one pass per round, several drafts


def test_prefix_cache_entry_cap_evicts_the_least_recently_used():
    from cuteafd_b200.runtime.paged import PagePool, SequenceTable
    from cuteafd_b200.runtime.prefix_cache import PrefixCache
    pool = PagePool(64)
    table = SequenceTable(pool)
    cache = PrefixCache(pool, table, max_pages=48)
    cache.max_entries = 2
    kept = []
    for i in range(4):
        s = table.new()
        table.reserve(s, 70)
        s.tokens, s.kv_len = [i] * 70, 70
        kept.append(cache.capture(s))
        table.free(s)
    assert len(cache.snapshots) == 2 and set(cache.snapshots) == {kept[2].sid, kept[3].sid}
    assert cache.lookup([0] * 70 + [9]).length == 0 and cache.lookup([3] * 70 + [9]).length == 70


def test_kv_pressure_stalls_by_default_and_ends_early_when_told_to():
    """Two long replies in a pool that holds only one to its end: by default the second stalls until the first has
    finished and both arrive whole; with an early-termination threshold the stalled one ends with ``length`` /
    ``kv_pressure`` once it has produced that many tokens."""
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)

    def serve(early):
        sched = Scheduler(OracleBackend(cfg, params, total_pages=9, prefill_chunk=64), max_active=2, reserve_chunk_tokens=64,
                          early_end_tokens=early)
        reqs = [Request(prompt=[3 + i] * 60, max_tokens=260, speculation=False) for i in range(2)]
        for r in reqs:
            sched.submit(r)
        done = {}
        for _ in range(4000):
            sched.step()
            for i, r in enumerate(reqs):
                while not r.events.empty():
                    ev = r.events.get()
                    if ev[0] == "done":
                        done[i] = (ev[1], ev[2]["completion_tokens"], ev[2].get("finish_detail", ""))
            if len(done) == 2:
                break
        return done, sched.stats.stalls
    whole, stalls = serve(-1)
    assert {v[1] for v in whole.values()} == {260} and all(v[2] == "" for v in whole.values()) and stalls > 0
    cut, _ = serve(20)
    kinds = sorted(v[2] for v in cut.values())
    assert kinds == ["", "kv_pressure"], cut
    short = next(v for v in cut.values() if v[2] == "kv_pressure")
    assert short[0] == "length" and 20 <= short[1] < 260
