"""The admission rule as a property: whatever mix of requests arrives and however the scheduler interleaves them, the
leases never exceed the pool, and the system never reaches a state where every admitted request is stalled (some
request can always run to its declared maximum and give its pages back).  Python and C++ forms take the same
decisions (rust/crates/cuteafd-engine/src/reserve.rs:1-32 states the rule)."""
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime.paged import PAGE
from cuteafd_b200.runtime.reserve import KvReserve, pages_for


def _forms():
    out = [lambda total, chunk: KvReserve(total, chunk)]
    try:
        from cuteafd_b200.runtime.native import NativeReserve, enabled
        if enabled():
            out.append(lambda total, chunk: NativeReserve(total, chunk))
    except Exception:                                              # noqa: BLE001 - optional on a CPU box
        pass
    return out


REQS = st.lists(st.tuples(st.integers(1, 3000), st.integers(1, 6000)), min_size=1, max_size=12)


@pytest.mark.parametrize("make", _forms())
@settings(max_examples=80, deadline=None)
@given(reqs=REQS, total=st.sampled_from([40, 96, 200]), chunk=st.sampled_from([128, 640, 2048]), order=st.randoms(use_true_random=False))
def test_some_request_can_always_finish(make, reqs, total, chunk, order):
    r = make(total, chunk)
    waiting = list(enumerate(reqs))
    active: dict[int, list[int]] = {}                 # rid -> [current length, final length]
    finished, spins = 0, 0
    while waiting or active:
        spins += 1
        assert spins < 20000, "no progress: the reserve let the system wedge"
        progressed = False
        # admission in arrival order; a refused head of the queue waits (no overtaking, as in the scheduler)
        while waiting:
            rid, (prompt, new) = waiting[0]
            if pages_for(prompt + new) > total:
                waiting.pop(0)                        # can never fit: refused outright by the front end
                finished += 1
                progressed = True
                continue
            if r.lease(rid, prompt, new) is None:
                break
            waiting.pop(0)
            active[rid] = [prompt, prompt + new]
            progressed = True
        # one decode step for the active requests, in a shuffled order
        ids = list(active)
        order.shuffle(ids)
        stalled = 0
        for rid in ids:
            cur, fin = active[rid]
            if r.needs_top_up(rid, cur + 1) and not r.top_up(rid):
                stalled += 1
                continue
            active[rid][0] = cur + min(PAGE, fin - cur)           # a page worth of tokens per step keeps the run short
            progressed = True
            if active[rid][0] >= fin:
                r.release(rid)
                del active[rid]
                finished += 1
        leased = sum(l.leased_pages for l in r.leases.values()) if hasattr(r, "leases") else r.leased
        assert leased <= total
        assert progressed or not active or stalled < len(ids), "every admitted request is stalled"
        if not progressed and not active and waiting:
            raise AssertionError("an empty system refused a request that fits")
    assert finished == len(reqs)
