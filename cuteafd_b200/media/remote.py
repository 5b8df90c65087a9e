"""Media towers on another process or host: the serving process keeps preprocessing, caching and placeholder expansion,
and sends patches / mel frames to an encoder service that holds the tower weights and answers with embedding rows.

    srv = EncoderServer(vision=VisionTower(...), audio=AudioTower(...)).start()        # where the towers live
    vision, audio = connect("127.0.0.1", srv.port)                                      # where requests are served
    MediaProcessor(vocab, hidden, vision, audio)                                         # proxies have the towers' interface

Frame: 4-byte big-endian header length, JSON header, raw tensor bytes.  Request header ``{"op": "hello" | "vision" |
"audio", "shape", "dtype", "grid"}``; reply ``{"ok", "shape", "dtype", "error"}``.  ``hello`` returns the towers'
configurations, which is all a proxy needs to answer ``cfg`` / ``rows_for`` locally.  One request in flight per
connection; a connection failure surfaces as ``MediaError`` on the request that hit it (media requests are independent,
so there is no latch: the next request reconnects).

Counterpart: the reference's encoder placement on another box (remote encoder over TCP, loader/media/ +
daemon/shared/media remote encoder).
"""
from __future__ import annotations

import dataclasses
import json
import socket
import struct
import threading

import torch

from .image import MediaError
from .towers import AudioTower, AudioTowerConfig, VisionTower, VisionTowerConfig

_DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}
MAX_HEADER, MAX_BODY = 1 << 16, 1 << 30


def _recv(sock: socket.socket, n: int) -> bytes:
    buf = bytearray()
    while len(buf) < n:
        chunk = sock.recv(min(n - len(buf), 1 << 20))
        if not chunk:
            raise ConnectionError("peer closed the connection")
        buf += chunk
    return bytes(buf)


def _send(sock: socket.socket, header: dict, t: torch.Tensor | None = None) -> None:
    body = b""
    if t is not None:
        t = t.contiguous().cpu()
        header = dict(header, shape=list(t.shape), dtype=str(t.dtype).replace("torch.", ""))
        body = t.view(torch.uint8).numpy().tobytes() if t.numel() else b""
    h = json.dumps(dict(header, bytes=len(body))).encode()
    sock.sendall(struct.pack(">I", len(h)) + h + body)


def _read(sock: socket.socket) -> tuple[dict, torch.Tensor | None]:
    (n,) = struct.unpack(">I", _recv(sock, 4))
    if n > MAX_HEADER:
        raise ConnectionError("oversized header")
    h = json.loads(_recv(sock, n))
    nb = int(h.get("bytes", 0))
    if nb > MAX_BODY:
        raise ConnectionError("oversized body")
    t = None
    if "shape" in h:
        # the header is not trusted: shape and dtype must describe exactly the bytes that follow, before anything is
        # allocated (the body itself is read either way, so the stream stays framed)
        raw = bytearray(_recv(sock, nb))
        shape, dt = h["shape"], _DT.get(h.get("dtype"))
        if (dt is None or not isinstance(shape, list) or len(shape) > 8
                or not all(isinstance(d, int) and not isinstance(d, bool) and d >= 0 for d in shape)):
            raise MalformedFrame("bad shape or dtype")
        count = 1
        for d in shape:
            count *= d
        if count * torch.empty(0, dtype=dt).element_size() != nb:
            raise MalformedFrame("shape and dtype do not match the body length")
        t = torch.frombuffer(raw, dtype=torch.uint8).view(dt).view(shape) if nb else torch.empty(shape, dtype=dt)
    return h, t


class MalformedFrame(ValueError):
    """A frame whose header and body disagree; the connection is still in step, so the peer gets an error reply."""


class EncoderServer:
    def __init__(self, vision: VisionTower | None = None, audio: AudioTower | None = None, host: str = "127.0.0.1", port: int = 0):
        self.vision, self.audio = vision, audio
        self.sock = socket.create_server((host, port))
        self.port = self.sock.getsockname()[1]
        self.encoded = 0
        self._stop = threading.Event()
        self._lock = threading.Lock()                       # one tower pass at a time
        self._t = threading.Thread(target=self._accept, name="media-encoder", daemon=True)

    def start(self) -> "EncoderServer":
        self._t.start()
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

    def _accept(self) -> None:
        while not self._stop.is_set():
            try:
                conn, _ = self.sock.accept()
            except OSError:
                return
            threading.Thread(target=self._serve, args=(conn,), daemon=True).start()

    def _serve(self, conn: socket.socket) -> None:
        try:
            while True:
                try:
                    h, t = _read(conn)
                except MalformedFrame as e:
                    _send(conn, {"ok": False, "error": f"malformed frame: {e}"})
                    continue
                except (ConnectionError, json.JSONDecodeError, struct.error, KeyError, ValueError, TypeError):
                    return
                op = h.get("op")
                try:
                    if op == "hello":
                        _send(conn, {"ok": True, "vision": dataclasses.asdict(self.vision.cfg) if self.vision else None,
                                     "audio": dataclasses.asdict(self.audio.cfg) if self.audio else None})
                    elif op == "vision" and self.vision is not None:
                        with self._lock:
                            out = self.vision.forward(t, tuple(h["grid"]))
                        self.encoded += 1
                        _send(conn, {"ok": True}, out)
                    elif op == "audio" and self.audio is not None:
                        with self._lock:
                            out = self.audio.forward(t)
                        self.encoded += 1
                        _send(conn, {"ok": True}, out)
                    else:
                        _send(conn, {"ok": False, "error": f"no tower for {op!r}"})
                except Exception as e:                      # noqa: BLE001 - reported to the client, the service stays up
                    _send(conn, {"ok": False, "error": f"{type(e).__name__}: {e}"})
        except OSError:
            pass
        finally:
            conn.close()


class _Link:
    def __init__(self, host: str, port: int, timeout: float):
        self.addr, self.timeout = (host, port), timeout
        self.sock: socket.socket | None = None
        self.lock = threading.Lock()

    def call(self, header: dict, t: torch.Tensor | None = None) -> tuple[dict, torch.Tensor | None]:
        with self.lock:
            try:
                if self.sock is None:
                    self.sock = socket.create_connection(self.addr, timeout=self.timeout)
                    self.sock.settimeout(self.timeout)
                _send(self.sock, header, t)
                h, out = _read(self.sock)
            except (OSError, ConnectionError, json.JSONDecodeError, struct.error) as e:
                if self.sock is not None:
                    self.sock.close()
                self.sock = None                            # the next request reconnects
                raise MediaError(f"media encoder at {self.addr[0]}:{self.addr[1]} unavailable: {e}") from e
        if not h.get("ok"):
            raise MediaError(f"media encoder refused: {h.get('error')}")
        return h, out


class RemoteVisionTower:
    def __init__(self, link: _Link, cfg: VisionTowerConfig):
        self.link, self.cfg = link, cfg

    def rows_for(self, grid: tuple[int, int]) -> int:
        return grid[0] * grid[1] // (self.cfg.merge ** 2)

    def forward(self, patches: torch.Tensor, grid: tuple[int, int]) -> torch.Tensor:
        return self.link.call({"op": "vision", "grid": list(grid)}, patches)[1]


class RemoteAudioTower:
    rows_for_frames = staticmethod(AudioTower.rows_for_frames)

    def __init__(self, link: _Link, cfg: AudioTowerConfig):
        self.link, self.cfg = link, cfg

    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        return self.link.call({"op": "audio"}, mel)[1]


def connect(host: str, port: int, timeout: float = 60.0):
    """(vision proxy or None, audio proxy or None) for the towers the service holds."""
    link = _Link(host, port, timeout)
    h, _ = link.call({"op": "hello"})
    v = RemoteVisionTower(link, VisionTowerConfig(**h["vision"])) if h.get("vision") else None
    a = RemoteAudioTower(_Link(host, port, timeout), AudioTowerConfig(**h["audio"])) if h.get("audio") else None
    return v, a
