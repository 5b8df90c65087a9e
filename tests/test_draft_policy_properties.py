"""The history draft policy as a property: under any sequence of outcomes its plans stay inside the block and the
request's room, always keep exactly one explore position while a position is still in doubt, and the row budget is
respected with every request keeping a prefix of what it asked for (rust/crates/cuteafd-core/src/draft_history.rs:1-120
gives the rules)."""
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime.speculation import DraftHistory, DrafterSpec

ROUND = st.tuples(st.integers(0, 3), st.integers(0, 12), st.integers(0, 12), st.booleans())


@settings(max_examples=150)
@given(block=st.integers(1, 8), copy=st.sampled_from([0, 0, 8, 32]), rounds=st.lists(ROUND, min_size=1, max_size=60))
def test_plans_stay_inside_block_and_room_and_outcomes_never_break_the_policy(block, copy, rounds):
    pol = DraftHistory(DrafterSpec(block, copy=copy))
    for rid, room, accepted, censored in rounds:
        plan = pol.plan(rid, room)
        assert 0 <= plan.keep <= min(block, room)
        if plan.explore is not None:
            assert plan.explore == plan.keep - 1                         # the one position past what history supports
        proposed = min(plan.keep, 1 + accepted % (block + 1))            # the drafter may offer fewer than asked
        plan = pol.refine(plan, proposed)
        assert plan.keep <= proposed
        if copy and plan.keep:
            plan.copy = min(copy, accepted % 5)
        took = min(accepted, plan.keep + plan.copy)
        pol.observe(plan, took, censored)
    life = pol.lifetime
    assert life["accepted"] <= life["proposed"] and life["rounds"] == len(rounds)
    for rid in range(4):
        pol.forget(rid)
    assert not pol.req


@settings(max_examples=200)
@given(asks=st.lists(st.tuples(st.integers(0, 8), st.integers(0, 6)), min_size=1, max_size=10), budget=st.integers(0, 40),
       probs=st.lists(st.floats(0, 1), min_size=14, max_size=14))
def test_row_budget_grants_prefixes(asks, budget, probs):
    from cuteafd_b200.runtime.speculation import Plan
    pol = DraftHistory(DrafterSpec(8, copy=8))
    plans = []
    for rid, (keep, cp) in enumerate(asks):
        p = Plan(rid, keep, None, list(probs))
        p.copy = cp if keep else 0
        plans.append(p)
    before = [(p.keep, p.copy) for p in plans]
    out = pol.settle(plans, budget)
    rows = sum(1 + p.keep + p.copy for p in out)
    assert rows <= max(budget, len(plans)) or rows == sum(1 + k + c for k, c in before) <= budget
    for (k0, c0), p in zip(before, out):
        assert 0 <= p.keep <= k0 and 0 <= p.copy <= c0
        assert p.copy == 0 or p.keep == k0                              # copy rows follow the whole neural draft only
