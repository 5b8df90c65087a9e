"""Expert wire protocol over TCP: frames, handshake, exact results against the whole oracle, failure latch."""
import socket
import struct
import zlib

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.parallel import wire
from cuteafd_b200.parallel.health import HealthError
from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights


def test_frame_layout_and_validation():
    req = wire.Request(wire.MOE, seq=7, layer=3, rows=2, hidden=4, routes=1, dtype=wire.F32, plan=b"p" * 16,
                       payload=b"\0" * (12 + 2 * 4 * 4))
    raw = req.pack()
    assert len(raw) == wire.HEADER + len(req.payload) and raw[:8] == b"CAFDWIRE"
    assert struct.unpack_from("<H", raw, 8)[0] == wire.VERSION and struct.unpack_from("<Q", raw, 16)[0] == 7
    assert struct.unpack_from("<Q", raw, 48)[0] == len(req.payload) and raw[60:76] == b"p" * 16
    got, nbytes, crc, status = wire.parse_request_header(raw[:wire.HEADER])
    assert status == wire.OK and (got.layer, got.rows, got.hidden, got.routes) == (3, 2, 4, 1) and crc == zlib.crc32(req.payload)
    bad = bytearray(raw[:wire.HEADER]); bad[0] = 0x58
    assert wire.parse_request_header(bytes(bad))[3] == wire.BAD_MAGIC
    bad = bytearray(raw[:wire.HEADER]); struct.pack_into("<H", bad, 8, 9)
    assert wire.parse_request_header(bytes(bad))[3] == wire.BAD_VERSION
    bad = bytearray(raw[:wire.HEADER]); struct.pack_into("<I", bad, 28, 3)           # rows disagree with the payload size
    assert wire.parse_request_header(bytes(bad))[3] == wire.BAD_SHAPE
    bad = bytearray(raw[:wire.HEADER]); struct.pack_into("<H", bad, 40, 77)
    assert wire.parse_request_header(bytes(bad))[3] == wire.BAD_DTYPE
    rsp = wire.Response(wire.MOE, wire.OK, 7, 1, 4, wire.F32, 1234, b"\1" * 16).pack()
    back, n, c = wire.parse_response_header(rsp[:wire.HEADER])
    assert (back.seq, back.rows, back.compute_us, n) == (7, 1, 1234, 16) and c == zlib.crc32(b"\1" * 16)
    assert wire.plan_hash({"a": 1, "b": 2}) == wire.plan_hash({"b": 2, "a": 1}) != wire.plan_hash({"a": 1, "b": 3})


def test_route_encoding_round_trip():
    g = torch.Generator().manual_seed(0)
    x = torch.randn(6, 8, generator=g).to(torch.bfloat16)
    idx = torch.tensor([[0, 5], [2, 3], [5, 1], [4, 4], [7, 6], [3, 2]])
    w = torch.rand(6, 2, generator=g)
    req, tok, slot = wire.encode_moe(1, 2, x, idx, w, 2, 5, b"h" * 16)
    assert req.routes == 6 and req.rows == 3 and tok.tolist() == [1, 1, 3, 3, 5, 5] and slot.tolist() == [0, 1, 0, 1, 0, 1]
    rows, row, sl, expert, weight = wire.decode_moe(req)
    assert torch.equal(rows, x[[1, 3, 5]]) and row.tolist() == [0, 0, 1, 1, 2, 2] and sl.tolist() == slot.tolist()
    assert expert.tolist() == [2, 3, 4, 4, 3, 2] and torch.allclose(torch.from_numpy(weight), w[[1, 1, 3, 3, 5, 5], [0, 1, 0, 1, 0, 1]])


@pytest.fixture()
def split():
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)
    dec = RefDecoder(cfg, params)
    plan = wire.plan_hash({"model": cfg.name, "experts": cfg.num_experts})
    half = cfg.num_experts // 2
    servers = []
    for lo, hi in ((0, half), (half, cfg.num_experts)):
        servers.append(wire.ExpertServer(wire.reference_compute(lambda layer, lo=lo, hi=hi: dec.expert_stack(layer, lo, hi), lo), plan).start())
    yield cfg, params, plan, servers, half
    for s in servers:
        s.stop()


def test_remote_experts_match_the_whole_model_exactly(split):
    cfg, params, plan, servers, half = split
    toks = torch.randint(0, cfg.vocab_size, (24,), generator=torch.Generator().manual_seed(3))
    whole = RefDecoder(cfg, params).forward(toks, KvState(cfg))
    remote = wire.RemoteExperts([("127.0.0.1", servers[0].port, 0, half), ("127.0.0.1", servers[1].port, half, cfg.num_experts)], plan)
    got = RefDecoder(cfg, params, moe_fn=remote).forward(toks, KvState(cfg))
    assert torch.equal(got, whole)                                     # same bits: the wire changes nothing
    assert servers[0].served > 0 and servers[1].served > 0 and all(l.pace_us for l in remote.links)
    remote.close()


def test_handshake_refuses_another_plan_and_latch_is_terminal(split):
    cfg, params, plan, servers, half = split
    with pytest.raises(HealthError, match="plan hash mismatch"):
        wire.ExpertLink("127.0.0.1", servers[0].port, wire.plan_hash({"other": 1}))
    assert servers[0].refused == 1
    link = wire.ExpertLink("127.0.0.1", servers[0].port, plan)
    assert link.call(wire.Request(wire.PING)).status == wire.OK
    servers[0].stop()
    link.sock.shutdown(socket.SHUT_RDWR)                               # the wire goes away under the link
    with pytest.raises(HealthError, match="expert link"):
        link.call(wire.Request(wire.PING))
    first = link.latch.reason
    with pytest.raises(HealthError) as e:                              # every later call refuses with the first reason
        link.call(wire.Request(wire.PING))
    assert str(e.value).endswith(first) and link.sock is None
    with pytest.raises(HealthError, match="connect"):
        wire.ExpertLink("127.0.0.1", 9, plan, timeout=0.5)


def test_server_checks_payload_and_dtype(split):
    cfg, params, plan, servers, half = split
    s = socket.create_connection(("127.0.0.1", servers[1].port), timeout=5)

    def ask(req_bytes):
        s.sendall(req_bytes)
        rsp, n, _ = wire.parse_response_header(wire.recv_exact(s, wire.HEADER))
        if n:
            wire.recv_exact(s, n)
        return rsp.status
    x = torch.randn(2, cfg.hidden).to(torch.bfloat16)
    idx = torch.full((2, cfg.top_k), half)
    req, _, _ = wire.encode_moe(1, cfg.first_dense_layers if hasattr(cfg, "first_dense_layers") else 1, x, idx,
                                torch.ones(2, cfg.top_k), half, cfg.num_experts, plan)
    assert ask(req.pack()) == wire.BAD_HASH                            # work before the handshake
    assert ask(wire.Request(wire.HELLO, plan=plan).pack()) == wire.OK
    raw = bytearray(req.pack()); raw[-1] ^= 0xFF                       # one payload byte flipped on the way
    assert ask(bytes(raw)) == wire.BAD_CRC
    servers[1].dtypes = {wire.F32}
    assert ask(req.pack()) == wire.BAD_DTYPE                           # ingress dtype validation
    servers[1].dtypes = {wire.BF16}
    assert ask(wire.Request(wire.PING).pack()) == wire.OK              # the connection survived the refusals
    bad = bytearray(wire.Request(wire.PING).pack()); bad[0] = 0
    assert ask(bytes(bad)) == wire.BAD_MAGIC                           # after this the server hangs up
    s.settimeout(2)
    assert s.recv(1) == b""
    s.close()


def test_expertd_tcp_worker_process(tmp_path):
    """``cuteafd expertd --tcp-port`` serves a snapshot's expert range to a remote decoder, bit for bit."""
    import subprocess
    import sys
    from cuteafd_b200.loader import load, snapshot
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="bf16", seed=7)
    procs, workers = [], []
    half = cfg.num_experts // 2
    try:
        for lo, hi in ((0, half), (half, cfg.num_experts)):
            p = subprocess.Popen([sys.executable, "-m", "cuteafd_b200.cli", "expertd", "--snapshot", src, "--tcp-port", "0",
                                  "--experts", f"{lo}:{hi}"], stdout=subprocess.PIPE, text=True)
            procs.append(p)
            line = p.stdout.readline()
            assert "expert worker" in line, line
            workers.append(("127.0.0.1", int(line.rsplit(":", 1)[1]), lo, hi))
        _, params = load.load_params(src, dtype=torch.bfloat16)
        toks = torch.arange(20) % cfg.vocab_size
        whole = RefDecoder(cfg, params).forward(toks, KvState(cfg))
        # each worker's plan hash covers its own range: one link per worker with its own hash
        links = []
        for h, port, lo, hi in workers:
            plan = wire.plan_hash({"model": cfg.name, "experts": cfg.num_experts, "range": [lo, hi]})
            links.append(wire.RemoteExperts([(h, port, lo, hi)], plan))

        def moe_fn(layer, x, idx, w):
            return sum(l(layer, x, idx, w) for l in links)
        got = RefDecoder(cfg, params, moe_fn=moe_fn).forward(toks, KvState(cfg))
        assert torch.equal(got, whole)
        for l in links:
            l.close()
    finally:
        for p in procs:
            p.kill()
            p.wait(timeout=10)


def test_injected_wire_fault_trips_the_latch_before_anything_is_sent(split):
    """The development fault site on the link: the request never leaves, the latch holds the reason, the worker saw
    nothing of the failed call."""
    from cuteafd_b200.utils.fault import ENABLE, PREFIX, FaultHooks
    cfg, params, plan, servers, half = split
    link = wire.ExpertLink("127.0.0.1", servers[0].port, plan)
    link.faults = FaultHooks(env={ENABLE: "1", PREFIX + "WIRE_SEND": "2"})
    link.faults.arm()
    assert link.call(wire.Request(wire.PING)).status == wire.OK
    with pytest.raises(HealthError, match="injected fault at WIRE_SEND"):
        link.call(wire.Request(wire.PING))
    assert not link.latch.ok and link.sock is None
    with pytest.raises(HealthError, match="injected fault"):           # terminal, like any other link failure
        link.call(wire.Request(wire.PING))


def test_serve_with_tcp_expert_workers(tmp_path, monkeypatch):
    """``serve --expert-workers`` on the host backend: replies equal the whole model's token for token, the profile
    modes report per-worker transport and compute time, an injected wire fault ends the step with a worker error."""
    from cuteafd_b200.cli import build_parser
    from cuteafd_b200.loader import snapshot
    from cuteafd_b200.runtime.scheduler import FAIL_WORKER, Request, collect
    from cuteafd_b200.serve.server import build_state
    cfg = tiny_moe()
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="bf16", seed=7)
    from cuteafd_b200.loader import load
    _, params = load.load_params(src)
    dec = RefDecoder(cfg, params)
    half = cfg.num_experts // 2
    servers = []
    for lo, hi in ((0, half), (half, cfg.num_experts)):
        plan = wire.plan_hash({"model": cfg.name, "experts": cfg.num_experts, "range": [lo, hi]})
        servers.append(wire.ExpertServer(wire.reference_compute(lambda layer, lo=lo, hi=hi: dec.expert_stack(layer, lo, hi), lo), plan).start())
    spec = ",".join(f"127.0.0.1:{s.port}:{lo}:{hi}" for s, (lo, hi) in zip(servers, ((0, half), (half, cfg.num_experts))))

    def run(state, prompt):
        r = Request(prompt, max_tokens=8, speculation=False)
        state.sched.submit(r)
        for _ in range(500):
            if not state.sched.step() and not state.sched.decoding and not state.sched.prefilling and not state.sched.pending and state.sched.waiting.empty():
                break
        return collect(r, timeout=1.0)
    try:
        base = ["serve", "--fake-engine", "--snapshot", src]
        whole = build_state(build_parser().parse_args(base))
        split = build_state(build_parser().parse_args(base + ["--expert-workers", spec, "--profile", "transport-timing,expert-timing"]))
        prompt = [3, 9, 27, 81, 5, 15]
        a, b = run(whole, prompt), run(split, prompt)
        assert a["tokens"] == b["tokens"] and b.get("error") is None
        rep = split.sched.profile.report()
        assert [w["experts"] for w in rep["transport"]] == [[0, half], [half, cfg.num_experts]]
        assert all(w["calls"] > 0 and w["round_trip"]["mean_us"] >= w["transport"]["mean_us"] >= 0 and w["sent_bytes"] > 0 for w in rep["transport"])
        assert rep["experts"]["imbalance"] >= 1.0 and all(w["compute"]["p99_us"] >= w["compute"]["p50_us"] for w in rep["experts"]["workers"])
        with pytest.raises(SystemExit, match="partition"):
            build_state(build_parser().parse_args(base + ["--expert-workers", f"127.0.0.1:{servers[0].port}:0:{half}"]))
        # the development wire fault: first expert call after readiness fails on the host; the latch is terminal
        monkeypatch.setenv("CUTEAFD_DEV_FAULT_HOOKS", "1")
        monkeypatch.setenv("CUTEAFD_DIAG_FAULT_WIRE_SEND", "1")
        faulty = build_state(build_parser().parse_args(base + ["--expert-workers", spec]))
        out = run(faulty, prompt)
        assert out["error"] and out["error"][0] == FAIL_WORKER and "injected fault at WIRE_SEND" in out["error"][1]
        assert not all(l.latch.ok for l in faulty.sched.be.remote_experts.links)
    finally:
        for s in servers:
            s.stop()
