"""The C++ host runtime against the Python forms on generated inputs: the sampler picks the same token from the same
row, parameters, seed and position; the draw is the same 24-bit uniform; the reserve takes the same decisions as the
Python reserve under any sequence of calls; the wire header parser classifies arbitrary bytes the same way."""
import numpy as np
import pytest
import torch
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.runtime import native as N
from cuteafd_b200.runtime.reserve import KvReserve
from cuteafd_b200.runtime.sampling import SamplingParams, select_token

pytestmark = pytest.mark.skipif(not N.enabled(), reason="the C++ runtime library is not built")

ROW = st.lists(st.floats(-12, 12, allow_nan=False, width=32), min_size=2, max_size=64)


@settings(max_examples=300)
@given(row=ROW, temperature=st.sampled_from([0.0, 0.2, 1.0, 1.9]), top_p=st.sampled_from([1.0, 0.95, 0.5, 0.01]),
       top_k=st.sampled_from([None, 1, 3, 50]), min_p=st.sampled_from([0.0, 0.1, 0.9]), seed=st.integers(0, 2 ** 62), pos=st.integers(0, 2 ** 31))
def test_sampler_forms_pick_the_same_token(row, temperature, top_p, top_k, min_p, seed, pos):
    x = torch.tensor(row, dtype=torch.float32)
    p = SamplingParams(temperature=temperature, top_p=top_p, top_k=top_k, min_p=min_p, seed=seed)
    assert N.sample_uniform(seed, pos) == p.uniform(pos)
    want = select_token(x, p, pos)
    got = N.sample_token(x, temperature, top_p, top_k, min_p, seed, pos)
    if got != want:
        # the two forms sum probabilities in a different order: a draw that lands within rounding of a boundary may fall
        # on either side of it, never further than the neighbouring entry of the order
        order = sorted(range(len(row)), key=lambda i: (-row[i], i))
        assert abs(order.index(got) - order.index(want)) == 1, (got, want)


OPS = st.lists(st.tuples(st.sampled_from(["lease", "top_up", "release", "grow"]), st.integers(0, 5), st.integers(1, 4000), st.integers(1, 4000)),
               min_size=1, max_size=60)


@settings(max_examples=150)
@given(ops=OPS, total=st.sampled_from([30, 120, 400]), chunk=st.sampled_from([64, 640, 4096]))
def test_reserve_forms_take_the_same_decisions(ops, total, chunk):
    a, b = KvReserve(total, chunk), N.NativeReserve(total, chunk)
    live: dict[int, int] = {}
    for op, rid, x, y in ops:
        if op == "lease" and rid not in live:
            ra, rb = a.lease(rid, x, y), b.lease(rid, x, y)
            assert (ra is not None) == bool(rb)
            if ra is not None:
                live[rid] = x
        elif rid in live:
            if op == "top_up":
                assert a.top_up(rid) == b.top_up(rid)
            elif op == "grow":
                live[rid] += x % 700
                assert a.needs_top_up(rid, live[rid]) == b.needs_top_up(rid, live[rid])
            elif op == "release":
                a.release(rid)
                b.release(rid)
                del live[rid]
        assert a.leased == b.leased and a.unleased == b.unleased


@settings(max_examples=300)
@given(raw=st.binary(min_size=96, max_size=96), fix_magic=st.booleans())
def test_wire_header_parsers_agree(raw, fix_magic):
    from cuteafd_b200.parallel import wire as W
    if fix_magic:
        raw = W.MAGIC + raw[8:]
    req, nbytes, crc, status = W.parse_request_header(raw)
    st_n, fields = N.wire_parse_request(raw)
    assert st_n == status
    if status == W.OK:
        assert (fields["rows"], fields["hidden"], fields["routes"], fields["payload_bytes"]) == (req.rows, req.hidden, req.routes, nbytes)
