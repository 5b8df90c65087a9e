"""WebSocket framing from the client's side of a socket pair: any text, cut into any fragments, masked with any key,
with pings in between and bytes arriving in any pieces, comes out of ``recv`` as the text that was sent; what the server
sends parses back by the lengths it wrote (RFC 6455 sections 5.2 - 5.4)."""
import io
import os
import socket
import struct
import threading

from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.serve import ws as W


def _frame(op: int, data: bytes, fin: bool, key: bytes) -> bytes:
    n = len(data)
    head = bytes([(0x80 if fin else 0) | op])
    if n < 126:
        head += bytes([0x80 | n])
    elif n < 1 << 16:
        head += bytes([0x80 | 126]) + struct.pack(">H", n)
    else:
        head += bytes([0x80 | 127]) + struct.pack(">Q", n)
    return head + key + bytes(b ^ key[i & 3] for i, b in enumerate(data))


def _read_server_frame(sock) -> tuple[int, bytes]:
    def exact(n):
        out = b""
        while len(out) < n:
            out += sock.recv(n - len(out))
        return out
    b0, b1 = exact(2)
    n = b1 & 0x7F
    assert not b1 & 0x80                              # a server never masks
    if n == 126:
        (n,) = struct.unpack(">H", exact(2))
    elif n == 127:
        (n,) = struct.unpack(">Q", exact(8))
    return b0 & 0x0F, exact(n)


@settings(max_examples=60)
@given(text=st.text(max_size=300), cuts=st.lists(st.integers(0, 2000), max_size=4), key=st.binary(min_size=4, max_size=4),
       ping_at=st.integers(0, 5), pieces=st.integers(1, 7), big=st.booleans())
def test_fragmented_masked_messages_with_pings_come_out_whole(text, cuts, key, ping_at, pieces, big):
    if big:
        text = text + "x" * 70000                     # forces the 64-bit length form
    raw = text.encode()
    pts = sorted({c % (len(raw) + 1) for c in cuts})
    frags, lo = [], 0
    for p in pts + [len(raw)]:
        frags.append(raw[lo:p])
        lo = p
    wire = b""
    for i, f in enumerate(frags):
        if i == ping_at % (len(frags) + 1):
            wire += _frame(W.OP_PING, b"hi", True, key)
        wire += _frame(W.OP_TEXT if i == 0 else 0, f, i == len(frags) - 1, key)
    a, b = socket.socketpair()
    try:
        server = W.Socket(io.BytesIO(b""), b.makefile("wb"), b)

        def feed():
            step = max(1, len(wire) // pieces)
            for i in range(0, len(wire), step):
                a.sendall(wire[i:i + step])
        t = threading.Thread(target=feed)
        t.start()
        got = server.recv()
        t.join()
        # (the byte-wise cut may split a character: the server decodes with replacement, as a browser would never send that)
        assert got == raw.decode("utf-8", "replace")
        if ping_at % (len(frags) + 1) < len(frags):
            assert _read_server_frame(a) == (W.OP_PONG, b"hi")
        server.send_json({"n": len(raw)})
        op, payload = _read_server_frame(a)
        assert op == W.OP_TEXT and payload == ('{"n": %d}' % len(raw)).encode()
        a.sendall(_frame(W.OP_CLOSE, struct.pack(">H", 1000), True, key))
        assert server.recv() is None and not server.open
    finally:
        a.close()
        b.close()


def test_unmasked_and_oversized_frames_close_the_connection():
    for wire, code in ((bytes([0x81, 2]) + b"hi", 1002), (bytes([0x81, 0x80 | 127]) + struct.pack(">Q", W.MAX_MESSAGE + 1), 1009)):
        a, b = socket.socketpair()
        try:
            server = W.Socket(io.BytesIO(b""), b.makefile("wb"), b)
            a.sendall(wire + os.urandom(4))
            try:
                server.recv()
                raise AssertionError("accepted")
            except W.Closed:
                pass
            op, payload = _read_server_frame(a)
            assert op == W.OP_CLOSE and struct.unpack(">H", payload[:2])[0] == code
        finally:
            a.close()
            b.close()
