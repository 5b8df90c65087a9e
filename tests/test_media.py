"""Media path on the CPU: preprocessing, towers, embedding cache, placeholder expansion, the oracle's embedding
override, prefix-cache separation of different images, and the HTTP surface with image / audio content parts."""
import base64
import io
import json
import struct
import wave

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.media import (AudioTower, AudioTowerConfig, MediaProcessor, VisionTower, VisionTowerConfig, decode_image,
                                preprocess_image, smart_resize)
from cuteafd_b200.media import audio as A
from cuteafd_b200.media.cache import EmbeddingCache
from cuteafd_b200.media.image import MediaError, bytes_from_url, patch_positions
from cuteafd_b200.media.processor import overrides_for, pseudo_id


def _png(h, w, seed=0) -> bytes:
    from PIL import Image
    g = torch.Generator().manual_seed(seed)
    px = torch.randint(0, 255, (h, w, 3), generator=g, dtype=torch.uint8).numpy()
    buf = io.BytesIO()
    Image.fromarray(px, "RGB").save(buf, format="PNG")
    return buf.getvalue()


def _wav(seconds=0.5, rate=8000, seed=0) -> bytes:
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(int(seconds * rate), generator=g) * 8000).clamp(-32000, 32000).to(torch.int16)
    buf = io.BytesIO()
    with wave.open(buf, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(rate)
        w.writeframes(struct.pack(f"<{x.numel()}h", *x.tolist()))
    return buf.getvalue()


def _towers(hidden):
    vc = VisionTowerConfig(width=64, depth=2, heads=4, mlp=128, out_hidden=hidden)
    ac = AudioTowerConfig(width=64, depth=1, heads=4, mlp=128, out_hidden=hidden)
    return VisionTower(vc, VisionTower.random_weights(vc)), AudioTower(ac, AudioTower.random_weights(ac))


def test_resize_and_patch_order():
    assert smart_resize(100, 150) == (112, 140)
    assert smart_resize(10, 10) == (56, 56)
    h, w = smart_resize(4000, 6000)
    assert h % 28 == 0 and w % 28 == 0 and h * w <= 1280 * 28 * 28
    with pytest.raises(MediaError):
        smart_resize(1, 500)
    px = decode_image(_png(60, 90))
    assert px.shape == (60, 90, 3)
    patches, (gh, gw) = preprocess_image(px)
    assert patches.shape == (gh * gw, 3 * 14 * 14) and gh % 2 == 0 and gw % 2 == 0
    pos = patch_positions(gh, gw)
    # the four patches of a merged cell are consecutive and form a 2 x 2 block
    cell = pos[:4]
    assert cell[:, 0].max() - cell[:, 0].min() == 1 and cell[:, 1].max() - cell[:, 1].min() == 1
    assert len({(int(r), int(c)) for r, c in pos}) == gh * gw


def test_data_urls_only():
    raw = _png(30, 30)
    url = "data:image/png;base64," + base64.b64encode(raw).decode()
    assert bytes_from_url(url) == raw
    with pytest.raises(MediaError):
        bytes_from_url("https://example.com/cat.png")
    with pytest.raises(MediaError):
        decode_image(b"not an image")


def test_towers_and_cache():
    vision, audio = _towers(32)
    mp = MediaProcessor(1000, 32, vision, audio, EmbeddingCache(1 << 20))
    k1, e1 = mp.encode_image(_png(60, 90, 1))
    k2, e2 = mp.encode_image(_png(60, 90, 2))
    k1b, e1b = mp.encode_image(_png(60, 90, 1))
    assert k1 != k2 and k1 == k1b and e1b is e1 and not torch.equal(e1, e2)
    assert e1.shape[1] == 32 and torch.isfinite(e1).all()
    assert mp.cache.hits == 1 and mp.encoded == 2
    mel = A.preprocess_audio(_wav())
    assert mel.shape[1] == 128
    _, ea = mp.encode_audio(_wav())
    assert ea.shape == (audio.rows_for_frames(mel.shape[0]), 32)
    small = EmbeddingCache(e1.numel() * e1.element_size() + 8)
    small.put(b"a", e1); small.put(b"b", e2)
    assert small.get(b"a") is None and small.get(b"b") is not None and small.evictions == 1


def test_expand_and_overrides():
    vision, audio = _towers(32)
    mp = MediaProcessor(1000, 32, vision, audio, start_id=7, end_id=8)
    enc = lambda s: [ord(c) % 256 for c in s]
    raw = _png(40, 40, 3)
    ids, spans = mp.expand(["ab", ("image", raw), "c", ("audio", _wav())], enc)
    assert len(spans) == 2 and ids[:2] == [97, 98] and ids[2] == 7
    s0 = spans[0]
    assert s0.start == 3 and ids[s0.start + s0.length] == 8
    assert all(t == pseudo_id(s0.key, 1000) for t in ids[s0.start:s0.start + s0.length]) and ids[s0.start] > 1000
    # a window that cuts through the first span
    rows, vals = overrides_for(spans, s0.start + 2, 4)
    n_in = min(4, s0.length - 2)
    assert rows[:n_in] == list(range(n_in)) and torch.equal(vals[:n_in], s0.embeds[2:2 + n_in])
    assert overrides_for(spans, 0, 2) is None


def test_oracle_takes_media_rows_and_prefix_cache_tells_images_apart():
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = tiny_moe()
    params = init_weights(cfg, seed=0)
    vision, _ = _towers(cfg.hidden)
    mp = MediaProcessor(cfg.vocab_size, cfg.hidden, vision)
    enc = lambda s: [ord(c) % 200 + 3 for c in s]
    prompts = [mp.expand(["look: ", ("image", _png(40, 40, seed)), " what is it?"], enc) for seed in (1, 2)]
    # oracle: override rows == running the decoder on hand-built input embeddings
    ids, spans = prompts[0]
    ref = RefDecoder(cfg, params)
    ov = overrides_for(spans, 0, len(ids))
    a = ref.forward(torch.tensor(ids), KvState(cfg), ov)
    other = list(ids)
    for r in ov[0]:
        other[r] = 5                                   # whatever id sits there does not matter
    b = ref.forward(torch.tensor(other), KvState(cfg), ov)
    assert torch.equal(a, b)
    c = ref.forward(torch.tensor(other), KvState(cfg))
    assert not torch.allclose(a, c)
    # scheduler + prefix cache: same text, different image -> different continuation source, no false cache hit
    be = OracleBackend(cfg, params, prefill_chunk=16)
    sched = Scheduler(be, max_active=2)
    outs = []
    for ids, spans in prompts + [prompts[0]]:
        req = Request(prompt=list(ids), max_tokens=4, media=spans)
        sched.submit(req)
        while True:
            sched.step()
            ev = req.events.get() if not req.events.empty() else None
            if ev and ev[0] in ("done", "error"):
                outs.append(ev)
                break
    assert all(o[0] == "done" for o in outs), outs
    assert outs[0][2]["cached_tokens"] == 0 and outs[1][2]["cached_tokens"] < len(prompts[1][0]) - 10
    assert outs[2][2]["cached_tokens"] >= 64 or len(prompts[0][0]) < 64      # the same image again restores its prefix


def test_http_accepts_image_and_audio_parts():
    import http.client
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.backends import OracleBackend
    from cuteafd_b200.runtime.scheduler import Scheduler
    from cuteafd_b200.serve import tokenizer
    from cuteafd_b200.serve.server import Server, ServerState
    cfg = tiny_moe()
    tok = tokenizer.ByteTokenizer(cfg.vocab_size)
    vision, audio = _towers(cfg.hidden)
    sched = Scheduler(OracleBackend(cfg, init_weights(cfg, seed=0)), max_active=2, eos_ids=tok.eos_ids)
    srv = Server(ServerState(sched, tok, cfg.name, media=MediaProcessor(cfg.vocab_size, cfg.hidden, vision, audio)), port=0).start()
    plain = Server(ServerState(Scheduler(OracleBackend(cfg, init_weights(cfg, seed=0)), eos_ids=tok.eos_ids), tok, cfg.name), port=0).start()

    def post(s, body):
        c = http.client.HTTPConnection("127.0.0.1", s.port, timeout=120)
        c.request("POST", "/v1/chat/completions", json.dumps(body).encode(), {"Content-Type": "application/json"})
        r = c.getresponse()
        out = (r.status, json.loads(r.read()))
        c.close()
        return out
    try:
        img = "data:image/png;base64," + base64.b64encode(_png(40, 56, 9)).decode()
        wav = base64.b64encode(_wav()).decode()
        body = {"max_tokens": 3, "temperature": 0, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "describe"}, {"type": "image_url", "image_url": {"url": img}},
            {"type": "input_audio", "input_audio": {"data": wav, "format": "wav"}}]}]}
        st, out = post(srv, body)
        assert st == 200 and out["usage"]["prompt_tokens"] > 20 and out["usage"]["completion_tokens"] >= 1
        st2, out2 = post(plain, body)
        assert st2 == 400 and "text only" in out2["error"]["message"]
        body["messages"][0]["content"][1]["image_url"]["url"] = "http://example.com/x.png"
        st3, out3 = post(srv, body)
        assert st3 == 400 and "data:" in out3["error"]["message"]
        c = http.client.HTTPConnection("127.0.0.1", srv.port, timeout=30)
        c.request("GET", "/v1/media")
        d = json.loads(c.getresponse().read())
        assert d["vision"] and d["audio"] and d["encoded"] == 2
    finally:
        srv.stop(); plain.stop()


def test_remote_encoder_gives_the_same_rows():
    """Towers behind the encoder service produce what local towers produce; a lost service is a media error on that
    request and the next request reconnects."""
    from cuteafd_b200.media.image import MediaError
    from cuteafd_b200.media.remote import EncoderServer, connect
    vision, audio = _towers(32)
    srv = EncoderServer(vision, audio).start()
    try:
        rv, ra = connect("127.0.0.1", srv.port)
        assert rv.cfg == vision.cfg and ra.cfg == audio.cfg and rv.rows_for((4, 6)) == vision.rows_for((4, 6))
        local = MediaProcessor(1000, 32, vision, audio)
        remote = MediaProcessor(1000, 32, rv, ra)
        png, wav = _png(60, 90, 3), _wav(seed=4)
        assert torch.equal(remote.encode_image(png)[1], local.encode_image(png)[1])
        assert torch.equal(remote.encode_audio(wav)[1], local.encode_audio(wav)[1])
        assert srv.encoded == 2
        only_v = EncoderServer(vision, None).start()
        v2, a2 = connect("127.0.0.1", only_v.port)
        assert a2 is None and v2 is not None
        only_v.stop()
        # a service that goes away: the request fails as a media error; against a live one the link reconnects
        rv.link.sock.close()
        rv.link.sock = None
        assert torch.equal(remote.encode_image(_png(60, 90, 5))[1], local.encode_image(_png(60, 90, 5))[1])
    finally:
        srv.stop()
    rv.link.sock.close(); rv.link.sock = None
    with pytest.raises(MediaError, match="unavailable"):
        remote.encode_image(_png(30, 30, 6))


def test_encoder_service_rejects_frames_whose_header_lies():
    """A header whose shape / dtype do not describe the body gets an error reply (nothing is allocated from it) and
    the connection keeps serving; an unknown dtype likewise."""
    import json
    import socket
    import struct
    from cuteafd_b200.media.remote import EncoderServer, _read
    vision, audio = _towers(32)
    srv = EncoderServer(vision, audio).start()
    try:
        with socket.create_connection(("127.0.0.1", srv.port), timeout=5) as c:
            def frame(header: dict, body: bytes = b""):
                h = json.dumps(dict(header, bytes=len(body))).encode()
                c.sendall(struct.pack(">I", len(h)) + h + body)
                return _read(c)[0]
            huge = frame({"op": "audio", "shape": [1 << 40, 1 << 20], "dtype": "float32"})      # no body at all
            assert huge["ok"] is False and "malformed" in huge["error"]
            short = frame({"op": "audio", "shape": [4, 4], "dtype": "float32"}, b"\0" * 12)
            assert short["ok"] is False and "malformed" in short["error"]
            odd = frame({"op": "audio", "shape": [3], "dtype": "complex999"}, b"\0" * 12)
            assert odd["ok"] is False
            assert frame({"op": "hello"})["ok"] is True                                          # still in step
    finally:
        srv.stop()


def test_encoderd_process_and_serve_flag(tmp_path):
    import subprocess
    import sys
    from cuteafd_b200.cli import build_parser
    from cuteafd_b200.serve.server import build_state
    p = subprocess.Popen([sys.executable, "-m", "cuteafd_b200.cli", "encoderd", "--random", "--hidden", "256", "--device", "cpu"],
                         stdout=subprocess.PIPE, text=True)
    try:
        line = p.stdout.readline()
        assert "media encoder (vision+audio)" in line, line
        port = int(line.rsplit(":", 1)[1])
        args = build_parser().parse_args(["serve", "--fake-engine", "--preset", "tiny-moe", "--media-encoder", f"127.0.0.1:{port}"])
        state = build_state(args)                              # tiny-moe has hidden 256: the towers' width fits
        assert state.media is not None and state.media.describe()["vision"] and state.media.describe()["audio"]
        key, rows = state.media.encode_image(_png(56, 56, 1))
        assert rows.shape[1] == 256 and torch.isfinite(rows).all()
    finally:
        p.kill()
        p.wait(timeout=10)
