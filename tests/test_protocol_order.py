"""Ordering fixtures for the flag protocols of the peer-memory kernels, on the CPU: every rank is a little program of
stores into peers' buffers, release-flag writes, acquire waits and reads; a scheduler interleaves the ranks in every
way a seed can produce, and a read must only ever see what the protocol says it sees (the reference keeps such
fixtures for its peer exchange: rust/crates/cuteafd-daemon/src/shared/peer_split/order/fixtures.rs).

The models are the protocols as the kernels run them: stores to a peer become visible no later than the flag written
after them (release / acquire), a rank's own operations run in program order, nothing else is ordered."""
import random

import pytest
from hypothesis import given, settings
from hypothesis import strategies as st


class World:
    def __init__(self, ranks: int):
        self.n = ranks
        self.buf: dict = {}          # (owner rank, buffer name) -> value last stored
        self.flag: dict = {}         # (owner rank, flag name) -> value
        self.reading: dict = {}      # (owner rank, buffer name) -> open read sections
        self.errors: list = []

    def run(self, programs, rng: random.Random, max_steps: int = 100000) -> None:
        live = {r: p for r, p in enumerate(programs)}
        pending = {r: next(p) for r, p in live.items()}
        for _ in range(max_steps):
            ready = [r for r, op in pending.items() if op[0] != "wait" or all(self.flag.get(k, 0) >= v for k, v in op[1])]
            if not ready:
                if pending:
                    self.errors.append(("deadlock", dict(pending)))
                return
            r = rng.choice(ready)
            op = pending[r]
            if op[0] == "store":                      # ("store", owner, name, value)
                key = (op[1], op[2])
                if self.reading.get(key):
                    self.errors.append(("store into a buffer that is being read", r, op))
                self.buf[key] = op[3]
            elif op[0] == "signal":                   # ("signal", owner, name, value)
                self.flag[(op[1], op[2])] = op[3]
            elif op[0] == "begin_read":               # ("begin_read", owner, name, expected)
                key = (op[1], op[2])
                if self.buf.get(key) != op[3]:
                    self.errors.append(("read saw", self.buf.get(key), "expected", op[3], r, op))
                self.reading[key] = self.reading.get(key, 0) + 1
            elif op[0] == "end_read":
                self.reading[(op[1], op[2])] -= 1
            try:
                pending[r] = next(live[r])
            except StopIteration:
                del pending[r], live[r]
        self.errors.append(("did not finish",))


def context_split_rank(me: int, n: int, layers: int, buffers: int):
    """parallel/context_split.py::DeviceContextSplit._exchange: partials into every rank's scratch (this turn's buffer),
    one flag per peer carrying the epoch, wait for every rank's flag, merge from the own scratch."""
    for layer in range(layers):
        b, epoch = layer % buffers, layer + 1
        for p in range(n):
            yield ("store", p, ("scratch", b, me), epoch)
        for p in range(n):
            yield ("signal", p, ("arrived", me), epoch)
        yield ("wait", [((me, ("arrived", r)), epoch) for r in range(n)])
        for r in range(n):
            yield ("begin_read", me, ("scratch", b, r), epoch)
        for r in range(n):
            yield ("end_read", me, ("scratch", b, r))


@settings(max_examples=150, deadline=None)
@given(seed=st.integers(0, 10 ** 9), n=st.sampled_from([2, 3, 4]), layers=st.integers(2, 7))
def test_context_split_with_two_scratch_buffers_never_tears(seed, n, layers):
    w = World(n)
    w.run([context_split_rank(r, n, layers, 2) for r in range(n)], random.Random(seed))
    assert not w.errors, w.errors[:3]


def test_one_scratch_buffer_would_tear_and_the_fixture_sees_it():
    """The reason for the second buffer: with one, a rank that is a layer ahead stores into the scratch a slower rank
    is still merging.  (Also shows the fixture can fail.)"""
    hit = 0
    for seed in range(200):
        w = World(2)
        w.run([context_split_rank(r, 2, 4, 1) for r in range(2)], random.Random(seed))
        hit += bool(w.errors)
    assert hit > 0


def afd_attention(me: int, experts: list[int], layers: int):
    """parallel/afd.py: per MoE layer the attention rank stores rows into every expert rank's slab, raises their dispatch
    flags, waits for every expert's done flag and reads its combine buffer."""
    for layer in range(layers):
        epoch = layer + 1
        for e in experts:
            yield ("store", e, ("slab", me), epoch)
        for e in experts:
            yield ("signal", e, ("dispatch", me), epoch)
        yield ("wait", [((me, ("done", e)), epoch) for e in experts])
        for e in experts:
            yield ("begin_read", me, ("combine", e), epoch)
        for e in experts:
            yield ("end_read", me, ("combine", e))


def afd_expert(me: int, sources: list[int], layers: int):
    """The expert rank serves the sources in rank order per layer: wait for the dispatch flag, read the slab (fc1), store
    the results into the source's combine buffer (fc2 epilogue), raise its done flag."""
    for layer in range(layers):
        epoch = layer + 1
        for s in sources:
            yield ("wait", [((me, ("dispatch", s)), epoch)])
            yield ("begin_read", me, ("slab", s), epoch)
            yield ("end_read", me, ("slab", s))
            yield ("store", s, ("combine", me), epoch)
            yield ("signal", s, ("done", me), epoch)


@settings(max_examples=150, deadline=None)
@given(seed=st.integers(0, 10 ** 9), sources=st.sampled_from([1, 2, 4]), experts=st.sampled_from([1, 2, 3]), layers=st.integers(1, 6))
def test_afd_exchange_single_buffers_are_safe_with_replicas(seed, sources, experts, layers):
    """One slab region and one combine buffer per (source, expert) pair suffice: a source cannot dispatch layer L + 1
    before it has every expert's done flag of layer L, and an expert raises that flag only after it has read the slab."""
    src, exp = list(range(sources)), list(range(sources, sources + experts))
    w = World(sources + experts)
    w.run([afd_attention(s, exp, layers) for s in src] + [afd_expert(e, src, layers) for e in exp], random.Random(seed))
    assert not w.errors, w.errors[:3]


def test_a_source_that_skips_the_done_wait_is_caught():
    def hasty(me, experts, layers):
        for op in afd_attention(me, experts, layers):
            if op[0] != "wait":
                yield op
    hit = 0
    for seed in range(100):
        w = World(2)
        w.run([hasty(0, [1], 3), afd_expert(1, [0], 3)], random.Random(seed))
        hit += bool(w.errors)
    assert hit > 0


def tp_rank(me: int, n: int, steps: int, layers: int):
    """parallel/tp.py + models/tp_gqa.py: one ``partials`` receive buffer and one ``x_full`` per rank, reused by every
    round of every layer.  Per step: wait until every rank released the previous step's buffers; push the first norm's
    rows; per layer the gathered rows are read by the qkv GEMM (which waits for the gather flags itself), the o
    projection stores partial rows at their owners and raises the reduce-scatter flags, the owner sums them, pushes
    norm2's rows with new gather flags, runs the FFN on its own rows, and pushes the next layer's rows without
    waiting for anybody; the head reads every row; the ready flags release the buffers."""
    epoch = 0
    for step in range(steps):
        if step:
            yield ("wait", [((me, ("ready", r)), epoch) for r in range(n)])
        epoch += 1
        tag = (step, 0, "ln1")
        for p in range(n):
            yield ("store", p, ("x", me), tag)
        for p in range(n):
            yield ("signal", p, ("ag", me), epoch)
        for layer in range(layers):
            yield ("wait", [((me, ("ag", r)), epoch) for r in range(n)])            # qkv GEMM over every rank's rows
            for r in range(n):
                yield ("begin_read", me, ("x", r), tag)
            for r in range(n):
                yield ("end_read", me, ("x", r))
            epoch += 1
            for p in range(n):                                                       # o projection: rows to their owners
                yield ("store", p, ("partials", me), (step, layer))
            for p in range(n):
                yield ("signal", p, ("rs", me), epoch)
            yield ("wait", [((me, ("rs", r)), epoch) for r in range(n)])            # owner adds the partials in rank order
            for r in range(n):
                yield ("begin_read", me, ("partials", r), (step, layer))
            for r in range(n):
                yield ("end_read", me, ("partials", r))
            mid = (step, layer, "ln2")
            for p in range(n):
                yield ("store", p, ("x", me), mid)
            for p in range(n):
                yield ("signal", p, ("ag", me), epoch)
            yield ("begin_read", me, ("x", me), mid)                                 # FFN of the owned rows
            yield ("end_read", me, ("x", me))
            epoch += 1
            tag = (step, layer + 1, "ln1")
            for p in range(n):                                                       # next layer's rows: nothing to wait for
                yield ("store", p, ("x", me), tag)
            for p in range(n):
                yield ("signal", p, ("ag", me), epoch)
        yield ("wait", [((me, ("ag", r)), epoch) for r in range(n)])                # the head reads every row
        for r in range(n):
            yield ("begin_read", me, ("x", r), tag)
        for r in range(n):
            yield ("end_read", me, ("x", r))
        for p in range(n):
            yield ("signal", p, ("ready", me), epoch)


@settings(max_examples=120, deadline=None)
@given(seed=st.integers(0, 10 ** 9), n=st.sampled_from([2, 3, 4]), steps=st.integers(1, 3), layers=st.integers(1, 4))
def test_tensor_parallel_rounds_reuse_one_buffer_safely(seed, n, steps, layers):
    w = World(n)
    w.run([tp_rank(r, n, steps, layers) for r in range(n)], random.Random(seed))
    assert not w.errors, w.errors[:3]


def test_without_the_step_boundary_handshake_the_next_step_overwrites_the_head_rows():
    def no_handshake(me, n, steps, layers):
        for op in tp_rank(me, n, steps, layers):
            if not (op[0] == "wait" and op[1] and op[1][0][0][1][0] == "ready"):
                yield op
    hit = 0
    for seed in range(200):
        w = World(2)
        w.run([no_handshake(r, 2, 3, 1) for r in range(2)], random.Random(seed))
        hit += bool(w.errors)
    assert hit > 0
