"""The expert wire format under generated inputs: any routing survives encode -> header -> decode unchanged, the header
parser classifies arbitrary bytes without raising, and a frame whose sizes do not add up is named, not trusted
(the reference fuzzes its transport the same way, all on loopback: transport/tests/upstream_fault_injection.rs:331-749)."""
import numpy as np
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.parallel import wire as W


@settings(max_examples=150, deadline=None)
@given(T=st.integers(1, 9), k=st.integers(1, 4), E=st.integers(2, 12), H=st.sampled_from([8, 32]), seed=st.integers(0, 99), cut=st.integers(0, 11))
def test_any_routing_round_trips(T, k, E, H, seed, cut):
    g = torch.Generator().manual_seed(seed)
    k = min(k, E)
    x = torch.randn(T, H, generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    w = torch.rand(T, k, generator=g)
    lo = min(cut, E - 1)
    hi = E
    req, tok, slot = W.encode_moe(7, 3, x, idx, w, lo, hi, b"p" * 16)
    raw = req.pack()
    head, nbytes, crc, status = W.parse_request_header(raw[:W.HEADER])
    assert status == W.OK and nbytes == len(raw) - W.HEADER
    head.payload = raw[W.HEADER:]
    rows, row, s, expert, weight = W.decode_moe(head)
    # every route in [lo, hi) arrives once, with its own row's data, slot and weight
    want = [(t, j) for t in range(T) for j in range(k) if lo <= int(idx[t, j]) < hi]
    assert len(row) == len(want) == len(tok)
    for n, (t, j) in enumerate(want):
        assert (int(tok[n]), int(slot[n]), int(s[n]), int(expert[n])) == (t, j, j, int(idx[t, j]))
        assert torch.equal(rows[row[n]], x[t]) and np.isclose(weight[n], float(w[t, j]))
    assert rows.shape[0] == len({t for t, _ in want})          # a row travels once however many of its routes land here


@settings(max_examples=300, deadline=None)
@given(raw=st.binary(min_size=W.HEADER, max_size=W.HEADER))
def test_arbitrary_header_bytes_are_classified_not_trusted(raw):
    req, nbytes, crc, status = W.parse_request_header(raw)
    assert status in range(len(W.STATUS_NAMES))
    if status == W.OK:
        assert raw[:8] == W.MAGIC and nbytes <= W.MAX_PAYLOAD
    try:
        W.parse_response_header(raw)
    except W.WireError:
        pass


@given(rows=st.integers(0, 50), hidden=st.integers(0, 64), routes=st.integers(0, 80), extra=st.integers(-5, 5))
def test_sizes_that_do_not_add_up_are_a_bad_shape(rows, hidden, routes, extra):
    n = routes * 12 + rows * hidden * 2 + extra
    if n < 0:
        return
    req = W.Request(W.MOE, 1, 0, 0, rows, hidden, routes, W.BF16, W.F32, 0, b"p" * 16, b"\0" * n)
    _, nbytes, _, status = W.parse_request_header(req.pack()[:W.HEADER])
    assert status == (W.OK if extra == 0 and hidden > 0 else W.BAD_SHAPE)
