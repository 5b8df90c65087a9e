"""The scheduler under generated request mixes on the oracle backend: whatever arrives in whatever order, with
speculation on or off, repeated prompts, cancels and a pool that is sometimes too small for everybody at once,
every request ends exactly once, greedy and seeded-sampling replies equal what the same prompt gives alone, and when the last request is
gone no page is left behind (free pages + pages the prefix cache holds = the pool).  The reference qualifies its
prefix cache with a multi-turn torture and leak accounting (scripts/qualify/qualify-prefix-cache.py)."""
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200 import tiny_moe
from cuteafd_b200.ref.model import init_weights
from cuteafd_b200.runtime.backends import OracleBackend
from cuteafd_b200.runtime.sampling import SamplingParams
from cuteafd_b200.runtime.scheduler import Request, Scheduler
from cuteafd_b200.runtime.speculation import NgramDrafter

CFG = tiny_moe()
PARAMS = init_weights(CFG, seed=0)
STEMS = [[5, 6, 7, 8] * 20, [9] * 70 + [3, 4] * 10, [11, 12, 13] * 9]
_ALONE: dict = {}


def _alone(prompt: tuple, n: int, params: SamplingParams) -> list[int]:
    """The reply the prompt gets on an empty server without drafts."""
    key = (prompt, n, params)
    if key not in _ALONE:
        s = Scheduler(OracleBackend(CFG, PARAMS, total_pages=64, prefill_chunk=64), max_active=1)
        r = s.submit(Request(prompt=list(prompt), max_tokens=n, speculation=False, cold=True, params=params))
        out = []
        for _ in range(2000):
            s.step()
            while not r.events.empty():
                ev = r.events.get()
                if ev[0] == "tokens":
                    out += ev[1]
                elif ev[0] == "done":
                    _ALONE[key] = out
                    return out
        raise AssertionError("the reference run did not end")
    return _ALONE[key]


REQ = st.tuples(st.integers(0, 2), st.integers(0, 30), st.integers(1, 9), st.booleans(), st.integers(0, 40), st.booleans())


@settings(max_examples=12, deadline=None)
@given(reqs=st.lists(REQ, min_size=1, max_size=7), pages=st.sampled_from([12, 20, 64]), active=st.integers(1, 4), cancel=st.integers(0, 10 ** 6),
       host_slots=st.sampled_from([0, 0, 16]))
def test_every_request_ends_once_with_the_reply_it_gets_alone_and_no_page_leaks(reqs, pages, active, cancel, host_slots):
    # (host_slots: a pinned tier behind the device cache, on a virtual clock: evicted snapshots spill and come back)
    be = OracleBackend(CFG, PARAMS, total_pages=pages, prefill_chunk=64, max_decode_rows=4, host_slots=host_slots)
    sched = Scheduler(be, max_active=active, queue_depth=32, drafter=NgramDrafter(block=3), reserve_chunk_tokens=64)
    live = []
    for stem, tail, n, spec, arrive, sample in reqs:
        prompt = STEMS[stem] + [20 + tail % 7] * (tail % 12)
        # a sampled request draws from (seed, position) alone: batching, drafts and cache hits may not move a token
        params = SamplingParams(temperature=0.9, top_k=5, seed=7 * stem + tail) if sample else SamplingParams()
        live.append([Request(prompt=prompt, max_tokens=n, speculation=spec, params=params), arrive, [], None, False])
    doomed = cancel % (len(live) + 1)                       # one request may be cancelled mid-flight (index len = nobody)
    submitted = 0
    for tick in range(6000):
        for item in live:
            if item[1] == tick or (tick > 45 and not item[4]):
                if not item[4]:
                    sched.submit(item[0])
                    item[4] = True
                    submitted += 1
        if doomed < len(live) and tick == 25 and live[doomed][4]:
            live[doomed][0].cancelled.set()
        sched.step()
        for item in live:
            while not item[0].events.empty():
                ev = item[0].events.get()
                if ev[0] == "tokens":
                    item[2] += ev[1]
                elif ev[0] in ("done", "error"):
                    assert item[3] is None, "a request ended twice"
                    item[3] = ev
        if submitted == len(live) and all(item[3] is not None for item in live):
            break
    assert all(item[3] is not None for item in live), [item[3] for item in live]
    for i, (req, _, toks, end, _) in enumerate(live):
        if end[0] == "error":
            # only a request that can never fit may be refused
            assert (len(req.prompt) + req.max_tokens + 63) // 64 > pages - 1, end
            continue
        if end[1] == "cancelled":
            assert i == doomed
            continue
        assert end[1] in ("length", "stop") and toks == _alone(tuple(req.prompt), req.max_tokens, req.params)[:len(toks)] and len(toks) == end[2]["completion_tokens"]
    # nothing is left behind: what is not free is held by the prefix cache's snapshots (a partial tail page that a
    # prompt snapshot and a turn snapshot both keep is one page)
    sched.step()
    held, stack = set(), [be.prefix.root]
    while stack:
        node = stack.pop()
        stack += list(node.children.values())
        held |= {c.page for c in node.children.values()} | {t.tail_page for t in node.tails.values()}
    assert be.pool.free_pages + len(held) == pages - 1, (be.pool.free_pages, sorted(held), pages)
    be.prefix.clear()
    assert be.pool.free_pages == pages - 1
