"""Expert wire protocol and its TCP transport: routed-expert work for ranks that are NOT in this box's NVSwitch domain.

Inside one box the exchange is peer memory and flags (``parallel/afd.py``); nothing is serialised.  A deployment that
spills experts onto another host needs a byte format, a handshake that proves both sides run the same plan, and a
transport that fails once and loudly.  This module is that path.  It is deliberately simple: host buffers over TCP,
one request in flight per connection; its job is correctness and failure semantics, not bandwidth.

Frame = fixed 96-byte header + payload.  Little endian.

    request header                                   response header
    0   8s  magic  b"CAFDWIRE"                        0   8s  magic
    8   H   version (2)                               8   H   version
    10  H   kind   HELLO / MOE / PING / BYE           10  H   kind (echo)
    12  I   flags  F_REDUCE: sum a row's routes       12  I   status  OK / BAD_MAGIC / BAD_VERSION / BAD_HASH /
    16  Q   seq                                                       BAD_SHAPE / BAD_DTYPE / BAD_CRC / FAILED
    24  I   layer                                     16  Q   seq (echo)
    28  I   rows      distinct rows in the payload    24  I   rows in the payload
    32  I   hidden                                    28  I   hidden
    36  I   routes    12-byte route entries           32  H   dtype
    40  H   dtype     of the rows (BF16 / F16 / F32)  34  H   reserved
    42  H   reply dtype                               36  Q   payload bytes
    44  I   unit      prefill unit / decode lane id   44  I   crc32 of the payload
    48  Q   payload bytes                             48  Q   compute microseconds (the worker's pace)
    56  I   crc32 of the payload                      56  40x reserved
    60  16s plan hash
    76  20x reserved

MOE payload = ``routes`` entries ``(u32 row | slot << 24, u32 expert id, f32 gate weight)`` followed by ``rows`` x
``hidden`` activations.  The reply carries one output row per route, in route order, already multiplied by the gate
weight (with ``F_REDUCE``: one row per distinct input row, the routes of a row summed in route order).

Failure semantics: every connection owns a ``HealthLatch``.  The first wire failure (short read, timeout, bad header,
non-OK status) trips it with the reason; every later call raises immediately with that reason; nothing reconnects.

Counterpart: rust/crates/cuteafd-transport/src/protocol_v2.rs (magic + version, 96-byte headers, 12-byte route
entries, worker pace in the reply), transport/lib.rs:14-30 (terminal health latch), the expertd TCP bootstrap and
plan-hash handshake (rust/crates/cuteafd-daemon/src/commands/expertd.rs).
"""
from __future__ import annotations

import hashlib
import socket
import struct
import threading
import time
import zlib
from dataclasses import dataclass

import numpy as np
import torch

from ..utils.fault import InjectedFault
from .health import HealthError, HealthLatch

MAGIC = b"CAFDWIRE"
VERSION = 2
HEADER = 96
HELLO, MOE, PING, BYE = 1, 2, 3, 4
F_REDUCE = 1
OK, BAD_MAGIC, BAD_VERSION, BAD_HASH, BAD_SHAPE, BAD_DTYPE, BAD_CRC, FAILED = range(8)
STATUS_NAMES = ("ok", "bad magic", "bad version", "plan hash mismatch", "bad shape", "bad dtype", "payload checksum mismatch",
                "worker failed")
BF16, F16, F32 = 1, 2, 3
_DTYPES = {BF16: torch.bfloat16, F16: torch.float16, F32: torch.float32}
_CODES = {v: k for k, v in _DTYPES.items()}
_REQ = struct.Struct("<8sHHIQIIIIHHIQI16s20x")
_RSP = struct.Struct("<8sHHIQIIHHQIQ40x")
assert _REQ.size == HEADER and _RSP.size == HEADER
MAX_PAYLOAD = 1 << 31


class WireError(RuntimeError):
    pass


def plan_hash(obj) -> bytes:
    """16-byte digest of whatever describes the deployment (model name, expert ranges, formats...)."""
    import json
    return hashlib.sha256(json.dumps(obj, sort_keys=True, default=str).encode()).digest()[:16]


@dataclass
class Request:
    kind: int
    seq: int = 0
    flags: int = 0
    layer: int = 0
    rows: int = 0
    hidden: int = 0
    routes: int = 0
    dtype: int = BF16
    reply_dtype: int = F32
    unit: int = 0
    plan: bytes = b"\0" * 16
    payload: bytes = b""

    def pack(self) -> bytes:
        return _REQ.pack(MAGIC, VERSION, self.kind, self.flags, self.seq, self.layer, self.rows, self.hidden, self.routes,
                         self.dtype, self.reply_dtype, self.unit, len(self.payload), zlib.crc32(self.payload), self.plan) + self.payload


@dataclass
class Response:
    kind: int
    status: int
    seq: int = 0
    rows: int = 0
    hidden: int = 0
    dtype: int = F32
    compute_us: int = 0
    payload: bytes = b""

    def pack(self) -> bytes:
        return _RSP.pack(MAGIC, VERSION, self.kind, self.status, self.seq, self.rows, self.hidden, self.dtype, 0,
                         len(self.payload), zlib.crc32(self.payload), self.compute_us) + self.payload


def parse_request_header(raw: bytes) -> tuple[Request, int, int, int]:
    """-> (request without payload, payload bytes, crc, status).  A non-OK status means: answer it and close."""
    magic, ver, kind, flags, seq, layer, rows, hidden, routes, dt, rdt, unit, nbytes, crc, plan = _REQ.unpack(raw)
    req = Request(kind, seq, flags, layer, rows, hidden, routes, dt, rdt, unit, plan)
    if magic != MAGIC:
        return req, 0, 0, BAD_MAGIC
    if ver != VERSION:
        return req, 0, 0, BAD_VERSION
    if nbytes > MAX_PAYLOAD:
        return req, 0, 0, BAD_SHAPE
    if kind == MOE:
        if dt not in _DTYPES or rdt not in _DTYPES:
            return req, nbytes, crc, BAD_DTYPE
        want = routes * 12 + rows * hidden * torch.empty((), dtype=_DTYPES[dt]).element_size()
        if nbytes != want or hidden == 0:
            return req, nbytes, crc, BAD_SHAPE
    return req, nbytes, crc, OK


def parse_response_header(raw: bytes) -> tuple[Response, int, int]:
    magic, ver, kind, status, seq, rows, hidden, dt, _, nbytes, crc, us = _RSP.unpack(raw)
    if magic != MAGIC or ver != VERSION:
        raise WireError("reply is not a wire frame of this version")
    if nbytes > MAX_PAYLOAD:
        raise WireError("reply announces an impossible payload")
    return Response(kind, status, seq, rows, hidden, dt, us), nbytes, crc


def _to_bytes(t: torch.Tensor) -> bytes:
    t = t.contiguous().cpu()
    return t.view(torch.uint8).numpy().tobytes() if t.numel() else b""


def _from_bytes(raw: bytes, dtype: torch.dtype, shape: tuple[int, ...]) -> torch.Tensor:
    if not raw:
        return torch.empty(shape, dtype=dtype)
    return torch.frombuffer(bytearray(raw), dtype=torch.uint8).view(dtype).view(shape)


def encode_moe(seq: int, layer: int, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor, lo: int, hi: int, plan: bytes,
               unit: int = 0, reduce: bool = False, reply_dtype: int = F32) -> tuple[Request, np.ndarray, np.ndarray]:
    """The request for the experts [lo, hi).  Returns (request, token row of every route, slot of every route)."""
    hit = (idx >= lo) & (idx < hi)
    tok, slot = hit.nonzero(as_tuple=True)                      # row-major: a row's routes stay in slot order
    rows_used, inverse = torch.unique(tok, return_inverse=True)
    if rows_used.numel() >= 1 << 24 or idx.shape[1] > 255:
        raise WireError("a request carries at most 2^24 rows and 255 slots per row")
    ent = np.zeros(tok.numel(), dtype=[("row", "<u4"), ("expert", "<u4"), ("weight", "<f4")])
    ent["row"] = inverse.numpy().astype(np.uint32) | (slot.numpy().astype(np.uint32) << 24)
    ent["expert"] = idx[tok, slot].numpy().astype(np.uint32)
    ent["weight"] = w[tok, slot].float().numpy()
    payload = ent.tobytes() + _to_bytes(x[rows_used])
    req = Request(MOE, seq, F_REDUCE if reduce else 0, layer, int(rows_used.numel()), x.shape[1], int(tok.numel()),
                  _CODES[x.dtype], reply_dtype, unit, plan, payload)
    return req, tok.numpy(), slot.numpy()


def decode_moe(req: Request) -> tuple[torch.Tensor, np.ndarray, np.ndarray, np.ndarray, np.ndarray]:
    """-> (rows [rows, hidden], route row index, route slot, route expert, route weight)."""
    ent = np.frombuffer(req.payload[: req.routes * 12], dtype=[("row", "<u4"), ("expert", "<u4"), ("weight", "<f4")])
    x = _from_bytes(req.payload[req.routes * 12:], _DTYPES[req.dtype], (req.rows, req.hidden))
    row = (ent["row"] & 0xFFFFFF).astype(np.int64)
    if req.routes and (row.max() >= req.rows):
        raise WireError("a route names a row that is not in the payload")
    return x, row, (ent["row"] >> 24).astype(np.int64), ent["expert"].astype(np.int64), ent["weight"].astype(np.float32)


# ---- transport ---------------------------------------------------------------------------------------
def recv_exact(sock: socket.socket, n: int) -> bytes:
    buf = bytearray(n)
    view, got = memoryview(buf), 0
    while got < n:
        k = sock.recv_into(view[got:], n - got)
        if k == 0:
            raise WireError(f"peer closed the connection after {got} of {n} bytes")
        got += k
    return bytes(buf)


class ExpertServer:
    """Serves the experts of one worker.  ``compute(layer, x, row, expert, weight) -> [routes, hidden] fp32`` returns
    the weighted output of every route."""

    def __init__(self, compute, plan: bytes, host: str = "127.0.0.1", port: int = 0, dtypes=(BF16, F16, F32)):
        self.compute, self.plan, self.dtypes = compute, plan, set(dtypes)
        self.sock = socket.create_server((host, port))
        self.port = self.sock.getsockname()[1]
        self._stop = threading.Event()
        self.served = 0
        self.refused = 0
        self._threads: list[threading.Thread] = []
        self._accept = threading.Thread(target=self._accept_loop, name="expert-server", daemon=True)

    def start(self) -> "ExpertServer":
        self._accept.start()
        return self

    def stop(self) -> None:
        self._stop.set()
        try:
            self.sock.shutdown(socket.SHUT_RDWR)            # wakes the thread blocked in accept()
        except OSError:
            pass
        try:
            self.sock.close()
        except OSError:
            pass

    def _accept_loop(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            t = threading.Thread(target=self._serve, args=(conn,), daemon=True)
            t.start()
            self._threads.append(t)

    def _serve(self, conn: socket.socket) -> None:
        conn.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
        greeted = False
        try:
            while not self._stop.is_set():
                try:
                    raw = recv_exact(conn, HEADER)
                except WireError:
                    return
                req, nbytes, crc, status = parse_request_header(raw)
                if status in (BAD_MAGIC, BAD_VERSION) or (status == BAD_SHAPE and nbytes == 0):
                    self.refused += 1
                    conn.sendall(Response(req.kind, status, req.seq).pack())
                    return                                          # the stream cannot be trusted any more
                req.payload = recv_exact(conn, nbytes) if nbytes else b""
                if status == OK and zlib.crc32(req.payload) != crc:
                    status = BAD_CRC
                if status == OK and req.kind == MOE and req.dtype not in self.dtypes:
                    status = BAD_DTYPE                              # ingress dtype validation
                if status == OK and req.kind in (HELLO, MOE) and req.plan != self.plan:
                    status = BAD_HASH
                if status == OK and req.kind == MOE and not greeted:
                    status = BAD_HASH                               # work before the handshake
                if status != OK:
                    self.refused += 1
                    conn.sendall(Response(req.kind, status, req.seq).pack())
                    if req.kind == HELLO:
                        return
                    continue
                if req.kind == HELLO:
                    greeted = True
                    conn.sendall(Response(HELLO, OK, req.seq).pack())
                elif req.kind == PING:
                    conn.sendall(Response(PING, OK, req.seq).pack())
                elif req.kind == BYE:
                    conn.sendall(Response(BYE, OK, req.seq).pack())
                    return
                elif req.kind == MOE:
                    conn.sendall(self._moe(req).pack())
                else:
                    conn.sendall(Response(req.kind, FAILED, req.seq).pack())
        except (OSError, WireError):
            return
        finally:
            conn.close()

    def _moe(self, req: Request) -> Response:
        t0 = time.perf_counter()
        try:
            x, row, slot, expert, weight = decode_moe(req)
            out = self.compute(req.layer, x, row, expert, weight).float()           # [routes, hidden]
            if req.flags & F_REDUCE:
                red = torch.zeros(req.rows, req.hidden)
                for r in range(req.routes):                                          # route order = slot order within a row
                    red[row[r]] += out[r]
                out = red
            out = out.to(_DTYPES[req.reply_dtype])
        except Exception:                                                            # noqa: BLE001 - reported, not raised
            return Response(MOE, FAILED, req.seq)
        self.served += 1
        return Response(MOE, OK, req.seq, out.shape[0], req.hidden, req.reply_dtype,
                        int((time.perf_counter() - t0) * 1e6), _to_bytes(out))


class ExpertLink:
    """One connection to one worker, with its latch."""

    def __init__(self, host: str, port: int, plan: bytes, timeout: float = 30.0):
        self.latch = HealthLatch()
        self.plan, self.seq = plan, 0
        self.pace_us: list[int] = []
        self.rtt_us: list[int] = []              # whole round trips of the same calls (send .. reply parsed)
        self.calls = self.sent_bytes = self.recv_bytes = 0
        self.lock = threading.Lock()
        try:
            self.sock = socket.create_connection((host, port), timeout=timeout)
            self.sock.setsockopt(socket.IPPROTO_TCP, socket.TCP_NODELAY, 1)
            self.sock.settimeout(timeout)
        except OSError as e:
            self.sock = None
            self.latch.trip(f"connect to {host}:{port} failed: {e}")
            raise HealthError(f"exchange unavailable: {self.latch.reason}") from e
        self.call(Request(HELLO, plan=plan))

    faults = None            # utils.fault.FaultHooks: a WIRE_SEND fault fails the link before the request leaves

    def call(self, req: Request) -> Response:
        with self.lock:
            self.latch.require()                                    # refuses after the first failure, with its reason
            self.seq += 1
            req.seq = self.seq
            try:
                if self.faults is not None:
                    self.faults.hit("WIRE_SEND")
                t0 = time.perf_counter()
                frame = req.pack()
                self.sock.sendall(frame)
                rsp, nbytes, crc = parse_response_header(recv_exact(self.sock, HEADER))
                rsp.payload = recv_exact(self.sock, nbytes) if nbytes else b""
                if zlib.crc32(rsp.payload) != crc:
                    raise WireError("reply payload checksum mismatch")
                if rsp.seq != req.seq:
                    raise WireError(f"reply {rsp.seq} does not answer request {req.seq}")
                if rsp.status != OK:
                    raise WireError(f"worker refused: {STATUS_NAMES[rsp.status] if rsp.status < len(STATUS_NAMES) else rsp.status}")
            except (OSError, WireError, struct.error, InjectedFault) as e:
                self.latch.trip(f"expert link: {e}")
                self.close()
                raise HealthError(f"exchange unavailable: {self.latch.reason}") from e
            if rsp.kind == MOE:
                self.pace_us.append(rsp.compute_us)
                self.rtt_us.append(int((time.perf_counter() - t0) * 1e6))
                del self.pace_us[:-256], self.rtt_us[:-256]
                self.calls, self.sent_bytes, self.recv_bytes = self.calls + 1, self.sent_bytes + len(frame), self.recv_bytes + HEADER + nbytes
            return rsp

    def close(self) -> None:
        if self.sock is not None:
            try:
                self.sock.close()
            except OSError:
                pass
            self.sock = None


class RemoteExperts:
    """``moe_fn`` for the decoders: sends every worker its routes (in parallel) and assembles [T, k, hidden] fp32."""

    def __init__(self, workers: list[tuple[str, int, int, int]], plan, timeout: float = 30.0):
        """workers: (host, port, first expert, end expert).  ``plan``: one hash for every worker, or
        ``plan(lo, hi) -> hash`` when each worker's hash covers its own range (what ``expertd --tcp-port`` announces)."""
        self.ranges = [(lo, hi) for _, _, lo, hi in workers]
        self.plans = [plan(lo, hi) if callable(plan) else plan for _, _, lo, hi in workers]
        self.links = [ExpertLink(h, p, pl, timeout) for (h, p, _, _), pl in zip(workers, self.plans)]
        self.plan = self.plans[0] if self.plans else b""

    def __call__(self, layer: int, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        T, k = idx.shape
        parts = torch.zeros(T, k, x.shape[1], dtype=torch.float32)
        errors: list[BaseException] = []

        def one(link: ExpertLink, lo: int, hi: int) -> None:
            try:
                req, tok, slot = encode_moe(0, layer, x, idx, w, lo, hi, link.plan)
                if req.routes == 0:
                    return
                rsp = link.call(req)
                out = _from_bytes(rsp.payload, _DTYPES[rsp.dtype], (rsp.rows, rsp.hidden)).float()
                parts[torch.from_numpy(tok), torch.from_numpy(slot)] = out
            except BaseException as e:                              # noqa: BLE001 - re-raised on the caller's thread
                errors.append(e)
        threads = [threading.Thread(target=one, args=(l, lo, hi)) for l, (lo, hi) in zip(self.links, self.ranges)]
        for t in threads:
            t.start()
        for t in threads:
            t.join()
        if errors:
            raise errors[0]
        return parts

    def timing(self) -> list[dict]:
        """Per worker, over its last 256 expert calls: the worker's own compute time (from the reply header), the round
        trip seen here, and their difference (serialisation + the wire + the worker's queue)."""
        def stats(v):
            if not v:
                return None
            s = sorted(v)
            return {"mean_us": round(sum(s) / len(s), 1), "p50_us": s[len(s) // 2], "p99_us": s[min(len(s) - 1, int(len(s) * 0.99))]}
        out = []
        for l, (lo, hi) in zip(self.links, self.ranges):
            wire_us = [max(0, r - c) for r, c in zip(l.rtt_us, l.pace_us)]
            out.append({"experts": [lo, hi], "ok": l.latch.ok, "calls": l.calls, "sent_bytes": l.sent_bytes, "recv_bytes": l.recv_bytes,
                        "compute": stats(l.pace_us), "round_trip": stats(l.rtt_us), "transport": stats(wire_us)})
        return out

    def close(self) -> None:
        for l in self.links:
            if l.latch.ok:
                try:
                    l.call(Request(BYE))
                except HealthError:
                    pass
            l.close()


def reference_compute(stack_of, lo: int):
    """``compute`` for ``ExpertServer`` on plain tensors: ``stack_of(layer) -> (gate, up, down)`` for the experts
    [lo, ...).  Same arithmetic and rounding as the oracle's local expert path, grouped by expert."""
    from ..ref import ops

    def compute(layer: int, x: torch.Tensor, row: np.ndarray, expert: np.ndarray, weight: np.ndarray) -> torch.Tensor:
        gate, up, down = stack_of(layer)
        out = torch.zeros(len(row), x.shape[1], dtype=torch.float32)
        for e in np.unique(expert):
            sel = np.nonzero(expert == e)[0]
            y = ops.swiglu_mlp(x[torch.from_numpy(row[sel])], gate[e - lo], up[e - lo], down[e - lo])
            out[torch.from_numpy(sel)] = y.to(x.dtype).float() * torch.from_numpy(weight[sel])[:, None]
        return out
    return compute


def cuda_compute(stack_of, lo: int, device, expert_ffn: int):
    """``compute`` for ``ExpertServer`` on a GPU: the request's routes are sorted by expert into an expert-major slab with
    tile tables, and the routed FFN runs on the tcgen05 expert-grouped GEMMs (fc1 + SwiGLU, then fc2 with its epilogue
    scattering every row back to its route slot), the same kernels the NVLink expert ranks run.  ``stack_of(layer) ->
    (gate, up, down)`` bf16 stacks [n, I, H] / [n, H, I] on ``device`` for the experts [lo, lo + n).  Rows come back as
    bf16-rounded expert outputs times the route weight, as from ``reference_compute``."""
    from ..ops import kernels as K
    from .moe_exchange import pick_tile_rows
    dev = torch.device(device)
    state: dict = {}

    def buffers(rows: int, tiles: int, H: int):
        cap = state.get("cap", (0, 0, 0))
        if rows > cap[0] or tiles > cap[1] or H != cap[2]:
            rows, tiles = max(rows, 2 * cap[0], 256), max(tiles, 2 * cap[1], 64)
            state.update(cap=(rows, tiles, H), slab=torch.zeros(rows, H, dtype=torch.bfloat16, device=dev),
                         hbuf=torch.zeros(rows, expert_ffn, dtype=torch.bfloat16, device=dev),
                         out=torch.zeros(rows, H, dtype=torch.bfloat16, device=dev))
        return state["slab"], state["hbuf"], state["out"], state["cap"][1]

    def compute(layer: int, x: torch.Tensor, row: np.ndarray, expert: np.ndarray, weight: np.ndarray) -> torch.Tensor:
        gate, up, down = stack_of(layer)
        n_exp, n, H = gate.shape[0], len(row), x.shape[1]
        if n == 0:
            return torch.zeros(0, H, dtype=torch.float32)
        tile = pick_tile_rows(max(1, n // max(1, len(np.unique(expert)))), 1, 1)
        order = np.argsort(expert, kind="stable")
        local = expert[order].astype(np.int64) - lo
        counts = np.bincount(local, minlength=n_exp)
        padded = (counts + tile - 1) // tile * tile
        seg = np.concatenate([[0], np.cumsum(padded)])
        first = np.concatenate([[0], np.cumsum(counts)])
        slab_row = seg[local] + (np.arange(n) - first[local])             # slab position of every sorted route
        total = int(seg[-1])
        tile_expert = np.repeat(np.arange(n_exp), padded // tile).astype(np.int32)
        tile_row0 = np.concatenate([seg[e] + tile * np.arange(padded[e] // tile) for e in range(n_exp)]).astype(np.int32)
        row_dst = np.full(total, -1, dtype=np.int32)
        row_dst[slab_row] = order                                          # fc2's epilogue stores slab row r at out[row_dst[r]]
        slab, hbuf, out, max_tiles = buffers(total, len(tile_expert), H)
        xs = x.to(device=dev, dtype=torch.bfloat16)
        slab[:total].zero_()
        slab[torch.from_numpy(slab_row).to(dev)] = xs[torch.from_numpy(row[order].astype(np.int64)).to(dev)]
        te = torch.zeros(max_tiles, dtype=torch.int32, device=dev); te[:len(tile_expert)] = torch.from_numpy(tile_expert).to(dev)
        t0 = torch.zeros(max_tiles, dtype=torch.int32, device=dev); t0[:len(tile_row0)] = torch.from_numpy(tile_row0).to(dev)
        nt = torch.tensor([len(tile_expert)], dtype=torch.int32, device=dev)
        rd = torch.from_numpy(row_dst).to(dev)
        K.grouped_linear(slab, gate, hbuf, te, t0, nt, max_tiles, tile, w_up=up)
        K.grouped_linear(hbuf, down, hbuf, te, t0, nt, max_tiles, tile, row_dst=rd, out_ptr=out.data_ptr(), ldo=H)
        y = out[:n].float() * torch.from_numpy(weight.astype(np.float32)).to(dev)[:, None]
        return y.cpu()
    return compute
