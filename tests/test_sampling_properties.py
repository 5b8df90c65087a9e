"""Properties of the exact sampler's oracle (the GPU kernel is compared against it row by row in test_sampling_gpu.py):
the selected token always lies in the support the filters define, the support is what the filter order says, the
draw depends on (seed, position) only, and speculative acceptance is prefix-match with the target's own tokens
(rust/crates/cuteafd-core/src/target_sampling.rs:9-47 states the rules)."""
import math

import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime.sampling import SamplingParams, accept_prefix, select_rows, select_token

LOGITS = st.lists(st.floats(-8, 8, allow_nan=False, width=32), min_size=2, max_size=40)
PARAMS = st.builds(SamplingParams, temperature=st.sampled_from([0.0, 0.3, 1.0, 1.7]), top_p=st.sampled_from([1.0, 0.9, 0.5, 0.05]),
                   top_k=st.sampled_from([None, 1, 2, 5, 100]), min_p=st.sampled_from([0.0, 0.05, 0.5]), seed=st.integers(0, 2 ** 40))


def _support(x: torch.Tensor, p: SamplingParams) -> list[int]:
    """The filter order written out naively."""
    if p.greedy:
        return [int(torch.argmax(x))]
    z = (x / p.temperature).double()
    ids = [i for i in range(len(z)) if z[i] >= z.max() + math.log(p.min_p)] if p.min_p > 0 else list(range(len(z)))
    ids.sort(key=lambda i: (-z[i].item(), i))
    if p.top_k is not None:
        ids = ids[:p.top_k]
    pr = torch.softmax(z[ids], 0)
    if p.top_p < 1.0:
        acc, keep = 0.0, 0
        for v in pr.tolist():
            keep += 1
            acc += v
            if acc >= p.top_p:
                break
        ids = ids[:keep]
    return ids


@settings(max_examples=300, deadline=None)
@given(vals=LOGITS, p=PARAMS, pos=st.integers(0, 10 ** 6))
def test_selected_token_lies_in_the_support_and_the_best_token_survives(vals, p, pos):
    x = torch.tensor(vals, dtype=torch.float32)
    sup = _support(x, p)
    tok = select_token(x, p, pos)
    best = int(torch.nonzero(x == x.max())[0])
    assert best in sup                                   # no filter removes the best token
    # boundary cases of top_p differ by one entry between a cumulative sum in float64 and this naive loop; the token
    # is then either in the naive support or the very next entry of the order
    z = sorted(range(len(vals)), key=lambda i: (-vals[i], i))
    assert tok in sup or (not p.greedy and z.index(tok) == len(sup)), (tok, sup)
    assert tok == select_token(x, p, pos)                # same (seed, position): same token
    if p.greedy:
        assert tok == best                               # lowest id among the maxima


@settings(max_examples=100, deadline=None)
@given(vals=LOGITS, p=PARAMS, pos=st.integers(0, 1000), pad=st.integers(1, 5))
def test_a_row_does_not_depend_on_the_rows_around_it(vals, p, pos, pad):
    x = torch.tensor(vals, dtype=torch.float32)
    alone = select_token(x, p, pos)
    batch = torch.stack([torch.roll(x, i) for i in range(pad)] + [x])
    toks, status = select_rows(batch, [SamplingParams(temperature=1.0, seed=7)] * pad + [p], list(range(pad)) + [pos])
    assert status[-1] == 0 and toks[-1] == alone


@settings(max_examples=100, deadline=None)
@given(vals=LOGITS, allowed=st.sets(st.integers(0, 39), min_size=1), p=PARAMS, pos=st.integers(0, 1000))
def test_the_mask_comes_first(vals, allowed, p, pos):
    x = torch.tensor(vals, dtype=torch.float32)
    mask = torch.zeros(len(vals), dtype=torch.bool)
    ids = [i for i in allowed if i < len(vals)]
    if not ids:
        return
    mask[ids] = True
    assert select_token(x, p, pos, mask) in ids


@given(sel=st.lists(st.integers(0, 9), min_size=1, max_size=9), flip=st.integers(0, 8))
def test_acceptance_is_the_longest_matching_prefix(sel, flip):
    draft = list(sel[:-1])
    n, bonus = accept_prefix(sel, draft)
    assert n == len(draft) and bonus == sel[-1]          # every draft right: all accepted, the bonus row's token follows
    if flip < len(draft):
        draft[flip] = (draft[flip] + 1) % 10
        n, bonus = accept_prefix(sel, draft)
        assert n == flip and bonus == sel[flip]          # first mismatch: the target's own token replaces it
