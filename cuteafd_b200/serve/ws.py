"""WebSocket endpoints of the serving process: ``/v1/realtime`` (text sessions) and ``/v1/responses`` over a socket.

The listener is the standard library's threaded HTTP server, so the server side of RFC 6455 is written out here: the
upgrade handshake, masked client frames (text, continuation, ping, pong, close), unmasked server frames.  One
connection is one thread; while a response is generating, the thread alternates between the request's event queue
and the socket, so a ``response.cancel`` (or a closed socket) stops generation at the next scheduler step.

Realtime sessions keep the conversation on the server: ``session.update`` sets instructions and sampling defaults,
``conversation.item.create`` appends a message, ``response.create`` runs the chat template over the whole
conversation and streams ``response.text.delta`` events; the assistant's reply becomes a conversation item.  Audio
buffers are refused with an ``error`` event (no audio tower is served).

Counterparts: rust/crates/cuteafd-api/src/gateway/realtime.rs:33-37 and gateway/responses.rs:38-45 (WebSocket
transport of the Responses API).
"""
from __future__ import annotations

import base64
import hashlib
import json
import queue
import select
import struct
import time
import uuid

from ..runtime.scheduler import FAIL_UNAVAILABLE
from . import api
from .tokenizer import StopStream, StreamDecoder

_GUID = b"258EAFA5-E914-47DA-95CA-C5AB0DC85B11"
OP_CONT, OP_TEXT, OP_BIN, OP_CLOSE, OP_PING, OP_PONG = 0x0, 0x1, 0x2, 0x8, 0x9, 0xA
MAX_MESSAGE = 16 << 20


class Closed(Exception):
    pass


def accept_key(key: str) -> str:
    return base64.b64encode(hashlib.sha1(key.encode() + _GUID).digest()).decode()


def wants_upgrade(headers) -> bool:
    return "websocket" in headers.get("Upgrade", "").lower() and "upgrade" in headers.get("Connection", "").lower()


class Socket:
    """Server side of one upgraded connection (rfile / wfile of the HTTP handler)."""

    def __init__(self, rfile, wfile, raw_socket):
        self.w, self.sock = wfile, raw_socket
        self.open = True
        # bytes the HTTP reader buffered past the request head (a client that did not wait for the 101)
        self.buf = bytearray()
        raw_socket.setblocking(False)
        try:
            early = rfile.read1(65536)
            if early:
                self.buf += early
        except (BlockingIOError, OSError, ValueError):
            pass
        finally:
            raw_socket.setblocking(True)

    def _exact(self, n: int) -> bytes:
        while len(self.buf) < n:
            try:
                chunk = self.sock.recv(65536)
            except (ConnectionResetError, OSError) as e:
                self.open = False
                raise Closed() from e
            if not chunk:
                self.open = False
                raise Closed()
            self.buf += chunk
        out = bytes(self.buf[:n])
        del self.buf[:n]
        return out

    def _frame(self) -> tuple[bool, int, bytes]:
        b0, b1 = self._exact(2)
        fin, op = bool(b0 & 0x80), b0 & 0x0F
        masked, n = bool(b1 & 0x80), b1 & 0x7F
        if n == 126:
            (n,) = struct.unpack(">H", self._exact(2))
        elif n == 127:
            (n,) = struct.unpack(">Q", self._exact(8))
        if n > MAX_MESSAGE:
            self.close(1009, "message too large")
            raise Closed()
        if not masked:                                   # a client must mask (RFC 6455 5.1)
            self.close(1002, "unmasked frame")
            raise Closed()
        key = self._exact(4)
        data = bytearray(self._exact(n))
        for i in range(n):
            data[i] ^= key[i & 3]
        return fin, op, bytes(data)

    def send(self, payload: bytes, op: int = OP_TEXT) -> None:
        n = len(payload)
        head = bytes([0x80 | op])
        if n < 126:
            head += bytes([n])
        elif n < 1 << 16:
            head += bytes([126]) + struct.pack(">H", n)
        else:
            head += bytes([127]) + struct.pack(">Q", n)
        try:
            self.w.write(head + payload)
            self.w.flush()
        except (BrokenPipeError, ConnectionResetError, OSError) as e:
            self.open = False
            raise Closed() from e

    def send_json(self, obj: dict) -> None:
        self.send(json.dumps(obj).encode())

    def close(self, code: int = 1000, reason: str = "") -> None:
        if self.open:
            self.open = False
            try:
                self.send(struct.pack(">H", code) + reason.encode()[:100], OP_CLOSE)
            except Closed:
                pass

    def readable(self, timeout: float = 0.0) -> bool:
        return bool(self.buf) or bool(select.select([self.sock], [], [], timeout)[0])

    def recv(self) -> str | None:
        """Next text message (continuations joined); None after a close frame."""
        parts: list[bytes] = []
        while True:
            fin, op, data = self._frame()
            if op == OP_PING:
                self.send(data, OP_PONG)
                continue
            if op == OP_PONG:
                continue
            if op == OP_CLOSE:
                self.close(1000)
                return None
            if op == OP_BIN:
                self.close(1003, "text frames only")
                return None
            parts.append(data)
            if sum(map(len, parts)) > MAX_MESSAGE:
                self.close(1009, "message too large")
                return None
            if fin:
                return b"".join(parts).decode("utf-8", "replace")


def upgrade(handler) -> Socket | None:
    """Answer the handshake on a ``BaseHTTPRequestHandler``; None (and a 400) when the request is not a valid upgrade."""
    key = handler.headers.get("Sec-WebSocket-Key", "")
    if not key or handler.headers.get("Sec-WebSocket-Version", "") != "13":
        handler.send_response(400)
        handler.send_header("Sec-WebSocket-Version", "13")
        handler.send_header("Content-Length", "0")
        handler.end_headers()
        return None
    handler.send_response(101, "Switching Protocols")
    handler.send_header("Upgrade", "websocket")
    handler.send_header("Connection", "Upgrade")
    handler.send_header("Sec-WebSocket-Accept", accept_key(key))
    proto = handler.headers.get("Sec-WebSocket-Protocol", "")
    if proto:
        handler.send_header("Sec-WebSocket-Protocol", proto.split(",")[0].strip())
    handler.end_headers()
    handler.wfile.flush()
    handler.close_connection = True
    return Socket(handler.rfile, handler.wfile, handler.connection)


def _eid() -> str:
    return "event_" + uuid.uuid4().hex[:20]


def _generate(state, ws: Socket, body: dict, flavor: str, on_text, cancel_types: tuple[str, ...]):
    """Submit a request and pump its events; returns ("done", finish, usage, text) | ("error", kind, message) |
    ("cancelled", text).  Client frames that arrive meanwhile are looked at for a cancel."""
    try:
        req = api.build_request(body, state.tok, state.sched.be.vocab_size, None, flavor, getattr(state, "media", None),
                                max_output_tokens=int(getattr(state, "extras", {}).get("max_output_tokens", 0) or 0))
    except api.BadRequest as e:
        return ("error", "invalid_request_error", str(e))
    if not state.sched.ready.is_set():
        return ("error", FAIL_UNAVAILABLE, "engine is starting")
    state.sched.submit(req)
    dec = StreamDecoder(state.tok)
    stopper = StopStream(getattr(req, "stop_texts", ()))       # stop strings end the reply before them, as over HTTP
    eos = set(getattr(state.tok, "eos_ids", ()))
    text: list[str] = []
    cancelled = False
    while True:
        try:
            ev = req.events.get(timeout=0.02)
        except queue.Empty:
            ev = None
        if not cancelled and ws.open and ws.readable(0.0):
            try:
                msg = ws.recv()
            except Closed:
                msg = None
            if msg is None:
                req.cancelled.set()
                cancelled = True
            else:
                try:
                    t = json.loads(msg).get("type", "")
                except (json.JSONDecodeError, AttributeError):
                    t = ""
                if t in cancel_types:
                    req.cancelled.set()
                    cancelled = True
        if ev is None:
            continue
        if ev[0] == "tokens":
            piece = stopper.push(dec.push([t for t in ev[1] if t not in eos]))
            if piece and not cancelled:
                text.append(piece)
                on_text(piece)
            if stopper.hit is not None:
                req.cancelled.set()
        elif ev[0] == "done":
            tail = stopper.push(dec.flush()) + stopper.flush()
            if tail and not cancelled:
                text.append(tail)
                on_text(tail)
            if stopper.hit is not None and not cancelled:
                return ("done", "stop", ev[2], "".join(text))
            if cancelled:
                return ("cancelled", "".join(text), ev[2])
            return ("done", ev[1], ev[2], "".join(text))
        else:
            if cancelled:
                return ("cancelled", "".join(text), {})
            return ("error", ev[1], ev[2])


# ---------------------------------------------------------------------------------------------- /v1/responses
def serve_responses(state, ws: Socket) -> None:
    while ws.open:
        try:
            msg = ws.recv()
        except Closed:
            return
        if msg is None:
            return
        try:
            ev = json.loads(msg)
            assert isinstance(ev, dict)
        except (json.JSONDecodeError, AssertionError):
            ws.send_json({"type": "error", "error": {"type": "invalid_request_error", "message": "messages must be JSON objects"}})
            continue
        if ev.get("type") != "response.create":
            ws.send_json({"type": "error", "error": {"type": "invalid_request_error",
                                                       "message": f"unsupported event {ev.get('type')!r}"}})
            continue
        body = ev.get("response") if isinstance(ev.get("response"), dict) else {k: v for k, v in ev.items() if k != "type"}
        model = body.get("model") or state.model_id
        rid = "resp_" + uuid.uuid4().hex[:24]
        try:
            with state.lock:
                body, conv = api.continue_session(body, getattr(state, "sessions", {}))
        except api.BadRequest as e:
            ws.send_json({"type": "error", "error": {"type": "invalid_request_error", "message": str(e)}})
            continue
        try:
            ws.send_json({"type": "response.created", "response": {"id": rid, "status": "in_progress", "model": model}})
            t0 = time.time()
            out = _generate(state, ws, body, "responses",
                            lambda s: ws.send_json({"type": "response.output_text.delta", "response_id": rid, "delta": s}),
                            ("response.cancel",))
            if out[0] == "done":
                obj = api.responses_object(model, out[3], out[1], out[2], rid)
                with state.lock:
                    state.responses[rid] = obj
                    if hasattr(state, "sessions"):
                        state.sessions[rid] = list(conv) + [{"role": "assistant", "content": out[3]}]
                if state.usage:
                    state.usage.record(model, "responses", out[2], time.time() - t0, out[1])
                ws.send_json({"type": "response.completed", "response": obj})
            elif out[0] == "cancelled":
                ws.send_json({"type": "response.cancelled", "response": {"id": rid, "status": "cancelled"}})
            else:
                ws.send_json({"type": "error", "error": {"type": out[1], "message": out[2]}})
        except Closed:
            return


# ---------------------------------------------------------------------------------------------- /v1/realtime
class RealtimeSession:
    def __init__(self, model: str):
        self.id = "sess_" + uuid.uuid4().hex[:20]
        self.model = model
        self.instructions = ""
        self.temperature: float | None = None
        self.max_tokens: int | None = None
        self.items: list[dict] = []          # {"id", "role", "text"}

    def describe(self) -> dict:
        return {"id": self.id, "object": "realtime.session", "model": self.model, "modalities": ["text"],
                "instructions": self.instructions, "temperature": self.temperature,
                "max_response_output_tokens": self.max_tokens if self.max_tokens is not None else "inf"}

    def update(self, s: dict) -> str | None:
        if "modalities" in s and any(m != "text" for m in s["modalities"]):
            return "only the text modality is served"
        if "instructions" in s:
            self.instructions = str(s["instructions"])
        if "temperature" in s:
            self.temperature = float(s["temperature"])
        if "max_response_output_tokens" in s:
            v = s["max_response_output_tokens"]
            self.max_tokens = None if v in ("inf", None) else int(v)
        return None

    def chat_body(self, override: dict) -> dict:
        msgs = []
        ins = override.get("instructions", self.instructions)
        if ins:
            msgs.append({"role": "system", "content": ins})
        msgs += [{"role": it["role"], "content": it["text"]} for it in self.items]
        body = {"model": self.model, "messages": msgs}
        mt = override.get("max_output_tokens", override.get("max_response_output_tokens", self.max_tokens))
        if mt not in (None, "inf"):
            body["max_tokens"] = int(mt)
        temp = override.get("temperature", self.temperature)
        if temp is not None:
            body["temperature"] = float(temp)
        return body


def _item_text(item: dict) -> str:
    c = item.get("content", [])
    if isinstance(c, str):
        return c
    return "".join(p.get("text", "") for p in c if isinstance(p, dict) and p.get("type") in ("input_text", "text", "output_text"))


def serve_realtime(state, ws: Socket, model: str | None = None) -> None:
    sess = RealtimeSession(model or state.model_id)

    def err(message: str, code: str = "invalid_request_error", event_id: str | None = None) -> None:
        ws.send_json({"type": "error", "event_id": _eid(),
                      "error": {"type": code, "message": message, "event_id": event_id}})

    try:
        ws.send_json({"type": "session.created", "event_id": _eid(), "session": sess.describe()})
        while ws.open:
            msg = ws.recv()
            if msg is None:
                return
            try:
                ev = json.loads(msg)
                assert isinstance(ev, dict)
            except (json.JSONDecodeError, AssertionError):
                err("messages must be JSON objects")
                continue
            t, cid = ev.get("type", ""), ev.get("event_id")
            if t == "session.update":
                why = sess.update(ev.get("session") or {})
                if why:
                    err(why, event_id=cid)
                else:
                    ws.send_json({"type": "session.updated", "event_id": _eid(), "session": sess.describe()})
            elif t == "conversation.item.create":
                item = ev.get("item") or {}
                if item.get("type", "message") != "message" or item.get("role") not in ("user", "assistant", "system"):
                    err("only message items with role user / assistant / system are served", event_id=cid)
                    continue
                rec = {"id": item.get("id") or "item_" + uuid.uuid4().hex[:20], "role": item["role"], "text": _item_text(item)}
                sess.items.append(rec)
                ws.send_json({"type": "conversation.item.created", "event_id": _eid(),
                              "item": {"id": rec["id"], "type": "message", "role": rec["role"], "status": "completed",
                                       "content": [{"type": "input_text", "text": rec["text"]}]}})
            elif t == "conversation.item.delete":
                before = len(sess.items)
                sess.items = [it for it in sess.items if it["id"] != ev.get("item_id")]
                if len(sess.items) == before:
                    err("no such item", event_id=cid)
                else:
                    ws.send_json({"type": "conversation.item.deleted", "event_id": _eid(), "item_id": ev.get("item_id")})
            elif t == "response.create":
                rid, iid = "resp_" + uuid.uuid4().hex[:24], "item_" + uuid.uuid4().hex[:20]
                ws.send_json({"type": "response.created", "event_id": _eid(),
                              "response": {"id": rid, "object": "realtime.response", "status": "in_progress", "output": []}})
                ws.send_json({"type": "response.output_item.added", "event_id": _eid(), "response_id": rid, "output_index": 0,
                              "item": {"id": iid, "type": "message", "role": "assistant", "status": "in_progress", "content": []}})
                ws.send_json({"type": "response.content_part.added", "event_id": _eid(), "response_id": rid, "item_id": iid,
                              "output_index": 0, "content_index": 0, "part": {"type": "text", "text": ""}})
                out = _generate(state, ws, sess.chat_body(ev.get("response") or {}), "openai",
                                lambda s: ws.send_json({"type": "response.text.delta", "event_id": _eid(), "response_id": rid,
                                                        "item_id": iid, "output_index": 0, "content_index": 0, "delta": s}),
                                ("response.cancel",))
                if out[0] == "error":
                    err(out[2], out[1], cid)
                    ws.send_json({"type": "response.done", "event_id": _eid(),
                                  "response": {"id": rid, "status": "failed", "output": []}})
                    continue
                text = out[3] if out[0] == "done" else out[1]
                usage = out[2] if isinstance(out[2], dict) else {}
                status = "completed" if out[0] == "done" else "cancelled"
                sess.items.append({"id": iid, "role": "assistant", "text": text})
                item = {"id": iid, "type": "message", "role": "assistant", "status": status,
                        "content": [{"type": "text", "text": text}]}
                ws.send_json({"type": "response.text.done", "event_id": _eid(), "response_id": rid, "item_id": iid,
                              "output_index": 0, "content_index": 0, "text": text})
                ws.send_json({"type": "response.output_item.done", "event_id": _eid(), "response_id": rid, "output_index": 0,
                              "item": item})
                ws.send_json({"type": "response.done", "event_id": _eid(),
                              "response": {"id": rid, "object": "realtime.response", "status": status, "output": [item],
                                           "usage": {"input_tokens": usage.get("prompt_tokens", 0),
                                                     "output_tokens": usage.get("completion_tokens", 0),
                                                     "total_tokens": usage.get("prompt_tokens", 0) + usage.get("completion_tokens", 0),
                                                     "input_token_details": {"cached_tokens": usage.get("cached_tokens", 0)}}}})
            elif t == "response.cancel":
                err("no response is in progress", event_id=cid)
            elif t.startswith("input_audio_buffer.") or t.startswith("output_audio_buffer."):
                err("audio is not served by this deployment", "unsupported_modality", cid)
            else:
                err(f"unknown event type {t!r}", event_id=cid)
    except Closed:
        return
