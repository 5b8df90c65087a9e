"""FLAC decoding in the C++ host runtime: the format specification's two worked examples (checked against the MD5 their
STREAMINFO carries), and streams written by a small encoder below that exercises what the examples do not (LPC, Rice2,
escaped and multiple partitions, 8 / 24-bit, mono, every stereo decorrelation, explicit block sizes, a metadata chain)."""
import hashlib
import io
import struct
import wave

import pytest
import torch

from cuteafd_b200.media import audio as A
from cuteafd_b200.media.image import MediaError

# RFC 9639, appendix D.1: one frame of one stereo sample, verbatim subframes with wasted bits
EXAMPLE_1 = bytes.fromhex("664c6143800000221000100000000f00000f0ac442f0000000013e84b41807dc690307586a3dad1a2e0f"
                          "fff869180000bf0358fd03128baa9a")
# appendix D.2: the two frames (16 + 3 samples; side stereo, fixed predictors, Rice partitions) and their STREAMINFO
EXAMPLE_2_INFO = bytes.fromhex("001000100000170000440ac442f000000013d5b0564975e98b8d8b930422757b8103")
EXAMPLE_2_FRAMES = bytes.fromhex(
    "fff86998000f9912086701623d1442998f5df70d6fe00c17caeb21000ee7a77a24a1590c1217b603097b784faa9a33d285e070ad5b1b4851"
    "b4010d99d2cd1a68f1e6b810" "fff869180102a402c382c40bc14a03ee48dd03b67c1330")


def raw_decode(data: bytes, cap: int = 1 << 20):
    import ctypes as C
    from cuteafd_b200._native import lib as native
    L = native.rt_lib()
    L.cafd_flac_info.argtypes = [C.c_char_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_uint64)]
    L.cafd_flac_decode.argtypes, L.cafd_flac_decode.restype = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_uint64], C.c_longlong
    rate, ch, bits, total = C.c_uint32(), C.c_int(), C.c_int(), C.c_uint64()
    rc = L.cafd_flac_info(data, len(data), rate, ch, bits, total)
    if rc:
        return rc, None, None
    out = torch.zeros(cap * ch.value, dtype=torch.int32)
    n = L.cafd_flac_decode(data, len(data), out.data_ptr(), cap)
    return n, (out[: max(n, 0) * ch.value].view(-1, ch.value) if n >= 0 else None), (rate.value, ch.value, bits.value, total.value)


def md5_of(pcm: torch.Tensor, bits: int) -> bytes:
    width = (bits + 7) // 8
    return hashlib.md5(b"".join(int(v).to_bytes(width, "little", signed=True) for v in pcm.flatten().tolist())).digest()


def test_specification_examples_decode_to_their_md5():
    n, pcm, info = raw_decode(EXAMPLE_1)
    assert n == 1 and info == (44100, 2, 16, 1) and pcm.tolist() == [[25588, 10416]]
    assert md5_of(pcm, 16) == EXAMPLE_1[26:42]
    chain = (b"fLaC" + b"\x00\x00\x00\x22" + EXAMPLE_2_INFO + b"\x03\x00\x00\x12" + bytes(16) + b"\x00\x10"
             + b"\x04\x00\x00\x08" + struct.pack("<I", 0) + struct.pack("<I", 0) + b"\x81\x00\x00\x06" + bytes(6))
    n, pcm, info = raw_decode(chain + EXAMPLE_2_FRAMES)
    assert n == 19 and info == (44100, 2, 16, 19)
    assert pcm[0].tolist() == [10372, 6070] and pcm[-1].tolist() == [-16054, -9410]
    assert md5_of(pcm, 16) == EXAMPLE_2_INFO[18:34]


# ---- a small encoder, for what the examples do not cover -------------------------------------------------------
class W:
    def __init__(self):
        self.bits = []

    def u(self, v, k):
        self.bits += [(v >> (k - 1 - i)) & 1 for i in range(k)]

    def s(self, v, k):
        self.u(v & ((1 << k) - 1), k)

    def unary(self, z):
        self.bits += [0] * z + [1]

    def align(self):
        self.bits += [0] * (-len(self.bits) % 8)

    def bytes(self):
        assert len(self.bits) % 8 == 0
        return bytes(int("".join(map(str, self.bits[i:i + 8])), 2) for i in range(0, len(self.bits), 8))


def crc(data, poly, width):
    c, top, mask = 0, 1 << (width - 1), (1 << width) - 1
    for byte in data:
        c ^= byte << (width - 8)
        for _ in range(8):
            c = ((c << 1) ^ poly) & mask if c & top else (c << 1) & mask
    return c


def rice(w, res, order, block, porder, k, rice2=False, escape_part=None):
    w.u(1 if rice2 else 0, 2); w.u(porder, 4)
    i = 0
    for p in range(1 << porder):
        count = (block >> porder) - (order if p == 0 else 0)
        part = res[i:i + count]; i += count
        if p == escape_part:
            w.u(31 if rice2 else 15, 5 if rice2 else 4)
            raw = max(v.bit_length() for v in part + [0]) + 1
            w.u(raw, 5)
            for v in part:
                w.s(v, raw)
            continue
        w.u(k, 5 if rice2 else 4)
        for v in part:
            z = (v << 1) if v >= 0 else ((-v) << 1) - 1
            w.unary(z >> k)
            if k:
                w.u(z & ((1 << k) - 1), k)


FIXED = {0: [], 1: [1], 2: [2, -1], 3: [3, -3, 1], 4: [4, -6, 4, -1]}


def subframe(w, x, bps, spec):
    kind = spec["kind"]
    wasted = spec.get("wasted", 0)
    if wasted:
        assert all(v % (1 << wasted) == 0 for v in x)
        x = [v >> wasted for v in x]; bps -= wasted
    block = len(x)

    def head(t):
        w.u(0, 1); w.u(t, 6); w.u(1 if wasted else 0, 1)
        if wasted:
            w.unary(wasted - 1)
    if kind == "constant":
        head(0); w.s(x[0], bps)
    elif kind == "verbatim":
        head(1)
        for v in x:
            w.s(v, bps)
    else:
        if kind == "fixed":
            order, coefs, shift = spec["order"], FIXED[spec["order"]], 0
            head(8 + order)
        else:
            coefs, shift, prec = spec["coefs"], spec["shift"], spec["precision"]
            order = len(coefs)
            head(31 + order)
        for v in x[:order]:
            w.s(v, bps)
        if kind == "lpc":
            w.u(prec - 1, 4); w.s(shift, 5)
            for c in coefs:
                w.s(c, prec)
        res = [x[i] - (sum(c * x[i - 1 - j] for j, c in enumerate(coefs)) >> shift) for i in range(order, block)]
        rice(w, res, order, block, spec.get("porder", 0), spec.get("k", 4), spec.get("rice2", False), spec.get("escape"))


def encode(channels, rate, bps, frames, mono_total=None):
    """channels: lists of ints; frames: [(block, stereo_mode, [subframe spec per channel], blocksize_code)]."""
    total = len(channels[0])
    pcm = torch.tensor(channels).T
    info = W()
    info.u(16, 16); info.u(65535, 16); info.u(0, 24); info.u(0, 24); info.u(rate, 20); info.u(len(channels) - 1, 3)
    info.u(bps - 1, 5); info.u(total if mono_total is None else mono_total, 36)
    out = b"fLaC" + b"\x80\x00\x00\x22" + info.bytes() + md5_of(pcm, bps)
    at, number = 0, 0
    for block, mode, specs, code in frames:
        w = W()
        w.u(0x3FFE, 14); w.u(0, 1); w.u(0, 1)
        w.u(code, 4); w.u(0, 4)                                   # sample rate: from STREAMINFO
        w.u({None: len(channels) - 1, "left_side": 8, "side_right": 9, "mid_side": 10}[mode], 4)
        w.u({8: 1, 12: 2, 16: 4, 20: 5, 24: 6}[bps], 3); w.u(0, 1)
        w.u(number, 8)                                            # frame number < 128: one byte
        if code == 6:
            w.u(block - 1, 8)
        elif code == 7:
            w.u(block - 1, 16)
        w.u(crc(w.bytes(), 0x07, 8), 8)
        chans = [c[at:at + block] for c in channels]
        widths = [bps] * len(channels)
        if mode == "left_side":
            chans = [chans[0], [l - r for l, r in zip(*chans)]]; widths[1] += 1
        elif mode == "side_right":
            chans = [[l - r for l, r in zip(*chans)], chans[1]]; widths[0] += 1
        elif mode == "mid_side":
            chans = [[(l + r) >> 1 for l, r in zip(*chans)], [l - r for l, r in zip(*chans)]]; widths[1] += 1
        for x, width, spec in zip(chans, widths, specs):
            subframe(w, x, width, spec)
        w.align()
        body = w.bytes()
        out += body + struct.pack(">H", crc(body, 0x8005, 16))
        at += block; number += 1
    assert at == total
    return out, pcm


def signal(n, bps, seed, smooth=True):
    g = torch.Generator().manual_seed(seed)
    amp = (1 << (bps - 1)) * 0.4
    t = torch.arange(n, dtype=torch.float64)
    x = amp * torch.sin(t * 0.05 + seed) + (amp * 0.02) * torch.randn(n, generator=g, dtype=torch.float64)
    return [int(v) for v in x.round().tolist()]


def test_every_subframe_kind_residual_coding_and_stereo_mode():
    L, R = signal(4096 + 1024 + 300, 16, 1), signal(4096 + 1024 + 300, 16, 2)
    lpc = {"kind": "lpc", "coefs": [1813, -921, 77, -12], "shift": 10, "precision": 12, "porder": 3, "k": 9}
    frames = [
        (4096, "mid_side", [dict(lpc), dict(lpc, rice2=True, k=17, porder=2, escape=1)], 12),
        (1024, "left_side", [{"kind": "fixed", "order": 2, "porder": 4, "k": 7}, {"kind": "fixed", "order": 4, "k": 8}], 10),
        (300, "side_right", [{"kind": "fixed", "order": 3, "k": 6, "escape": 0}, {"kind": "fixed", "order": 0, "k": 13}], 7),
    ]
    data, pcm = encode([L, R], 48000, 16, frames)
    n, got, info = raw_decode(data)
    assert n == len(L) and info == (48000, 2, 16, len(L)) and torch.equal(got, pcm.to(torch.int32))
    # 24-bit mono: constant, verbatim and wasted bits; explicit 8-bit block size
    M = [5 << 8] * 192 + [v << 4 for v in signal(256, 20, 3)] + signal(77, 24, 4)
    data, pcm = encode([M], 96000, 24, [(192, None, [{"kind": "constant", "wasted": 8}], 1),
                                          (256, None, [{"kind": "fixed", "order": 1, "k": 12, "wasted": 4}], 8),
                                          (77, None, [{"kind": "verbatim"}], 6)])
    n, got, info = raw_decode(data)
    assert n == len(M) and info == (96000, 1, 24, len(M)) and torch.equal(got[:, 0], torch.tensor(M, dtype=torch.int32))
    # 8-bit independent stereo, order-1 LPC with a negative coefficient
    a, b = signal(576, 8, 5), signal(576, 8, 6)
    data, pcm = encode([a, b], 8000, 8, [(576, None, [{"kind": "lpc", "coefs": [-3], "shift": 2, "precision": 3, "k": 5},
                                                       {"kind": "fixed", "order": 2, "k": 3}], 2)])
    n, got, _ = raw_decode(data)
    assert n == 576 and torch.equal(got, pcm.to(torch.int32))


def test_damage_is_an_error_not_silence():
    L = signal(1024, 16, 7)
    data, _ = encode([L], 16000, 16, [(1024, None, [{"kind": "fixed", "order": 2, "k": 8}], 10)])
    assert raw_decode(data)[0] == 1024
    flipped = bytearray(data); flipped[len(data) // 2] ^= 0x10
    assert raw_decode(bytes(flipped))[0] < 0                                   # frame checksum (or the coding) refuses
    head = bytearray(data); head[42 + 2] ^= 0x01                               # inside the frame header: its own CRC-8
    assert raw_decode(bytes(head))[0] < 0
    assert raw_decode(data[:-40])[0] < 0 and raw_decode(b"fLaX" + data[4:])[0] == -1
    assert raw_decode(data[:30])[0] == -3 and raw_decode(data, cap=1000)[0] == -8
    for bad in (bytes(flipped), data[:-40], b"fLaC"):
        with pytest.raises(MediaError, match="cannot decode audio"):
            A.decode_flac(bad)


def wav_bytes(x: torch.Tensor, rate: int) -> bytes:
    b = io.BytesIO()
    with wave.open(b, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(rate)
        w.writeframes((x * 32767).round().to(torch.int16).numpy().tobytes())
    return b.getvalue()


def test_flac_and_wav_of_the_same_clip_give_the_same_features():
    L = signal(16000, 16, 9)
    flac, _ = encode([L], 16000, 16, [(4096, None, [{"kind": "fixed", "order": 2, "k": 9}], 12)] * 3
                     + [(16000 - 3 * 4096, None, [{"kind": "fixed", "order": 2, "k": 9}], 7)])
    x, rate = A.decode_audio(flac)
    assert rate == 16000 and x.shape == (16000,) and torch.equal(x, torch.tensor(L, dtype=torch.float32) / 32768.0)
    w, _ = A.decode_audio(wav_bytes(torch.tensor(L, dtype=torch.float32) / 32767.0, 16000))
    assert (w - x).abs().max() < 1e-3 and A.preprocess_audio(flac).shape == A.preprocess_audio(wav_bytes(x, 16000)).shape
    # a stream that does not declare its length (a streaming encoder) is counted first, then decoded
    live, _ = encode([L[:4096]], 16000, 16, [(4096, None, [{"kind": "fixed", "order": 2, "k": 9}], 12)], mono_total=0)
    y, _ = A.decode_audio(live)
    assert torch.equal(y, x[:4096])
    stereo, _ = encode([L[:576], [-v for v in L[:576]]], 16000, 16, [(576, "mid_side", [{"kind": "fixed", "order": 2, "k": 9}] * 2, 2)])
    assert A.decode_audio(stereo)[0].abs().max() == 0                          # channels are averaged
    with pytest.raises(MediaError, match="mp3"):
        A.decode_audio(b"ID3\x03" + bytes(64))
    with pytest.raises(MediaError, match="mp3"):
        A.decode_audio(b"\xff\xfb\x90\x00" + bytes(64))
    with pytest.raises(MediaError, match="neither"):
        A.decode_audio(b"OggS" + bytes(64))


def test_clip_and_request_bounds():
    """A clip of more than 300 s is refused from its header; a request is bounded in clips and in summed seconds."""
    from cuteafd_b200.media.processor import MediaProcessor
    long, _ = encode([[0] * 16], 8000, 16, [(16, None, [{"kind": "constant"}], 6)], mono_total=8000 * 301)
    with pytest.raises(MediaError, match="longer than 300"):
        A.decode_flac(long)

    class Tower:
        def forward(self, mel):
            return torch.zeros(2, 8)
    mp = MediaProcessor(1000, 8, audio=Tower())
    clips = [wav_bytes(torch.full((8000 * 2,), 0.001 * (i + 1)), 8000) for i in range(5)]
    ids, spans = mp.expand(["hi"] + [("audio", c) for c in clips[:4]], lambda s: [1])
    assert len(spans) == 4
    with pytest.raises(MediaError, match="more than 4 audio clips"):
        mp.expand([("audio", c) for c in clips], lambda s: [1])
    minutes = [wav_bytes(torch.full((100 * 250,), 0.001 * (i + 1)), 100) for i in range(3)]      # 250 s each at 100 Hz
    mp.expand([("audio", c) for c in minutes[:2]], lambda s: [1])
    with pytest.raises(MediaError, match="more than 600 seconds"):
        mp.expand([("audio", c) for c in minutes], lambda s: [1])
    with pytest.raises(MediaError, match="more than 600 seconds"):                               # cached clips still count
        mp.expand([("audio", c) for c in minutes], lambda s: [1])


def test_damaged_streams_never_read_or_write_out_of_bounds():
    """Request audio is untrusted input to native code: thousands of bit flips, byte splices and truncations of valid
    streams must each come back as a count within the caller's bound or as an error code (the buffer's guard words stay
    intact), never as a crash."""
    import ctypes as C
    import random

    from cuteafd_b200._native import lib as native
    L = native.rt_lib()
    L.cafd_flac_decode.argtypes, L.cafd_flac_decode.restype = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_uint64], C.c_longlong
    L.cafd_flac_decode_mono.argtypes, L.cafd_flac_decode_mono.restype = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_uint64], C.c_longlong
    a, b = signal(2304, 16, 11), signal(2304, 16, 12)
    lpc = {"kind": "lpc", "coefs": [1500, -700, 90], "shift": 10, "precision": 12, "porder": 2, "k": 8}
    seeds = [encode([a, b], 44100, 16, [(1152, "mid_side", [dict(lpc), dict(lpc, rice2=True, escape=2)], 3),
                                         (1152, "left_side", [{"kind": "fixed", "order": 3, "k": 7, "porder": 3}, {"kind": "verbatim"}], 3)])[0],
             encode([a[:700]], 8000, 16, [(700, None, [{"kind": "fixed", "order": 4, "k": 6, "wasted": 0}], 7)])[0],
             EXAMPLE_1, b"fLaC\x80\x00\x00\x22" + EXAMPLE_2_INFO + EXAMPLE_2_FRAMES]
    cap, guard = 2304, 0x5A5A5A5A
    ints = torch.full((cap * 2 + 64,), guard, dtype=torch.int32)
    floats = torch.full((cap + 64,), 7.25, dtype=torch.float32)
    rng = random.Random(5)
    outcomes = {"ok": 0, "error": 0}
    for trial in range(4000):
        d = bytearray(rng.choice(seeds))
        for _ in range(rng.randint(1, 4)):
            kind = rng.random()
            at = rng.randrange(4, len(d))
            if kind < 0.6:
                d[at] ^= 1 << rng.randrange(8)
            elif kind < 0.8:
                d[at:at + rng.randint(1, 8)] = bytes(rng.randrange(256) for _ in range(rng.randint(0, 8)))
            else:
                del d[at:]
            if len(d) < 8:
                break
        raw = bytes(d)
        n = L.cafd_flac_decode(raw, len(raw), ints.data_ptr(), cap)
        m = L.cafd_flac_decode_mono(raw, len(raw), floats.data_ptr(), cap)
        assert n == m and n <= cap
        outcomes["ok" if n >= 0 else "error"] += 1
        assert ints[cap * 2:].eq(guard).all() and floats[cap:].eq(7.25).all()
    assert outcomes["error"] > 3000 and outcomes["ok"] > 0, outcomes          # CRCs catch nearly everything; metadata hits pass


def test_a_flac_clip_through_the_chat_api_matches_the_same_clip_as_wav():
    """``input_audio`` with FLAC bytes reaches the audio tower as the same samples a WAV of the clip gives: same
    prompt length, same reply."""
    import base64

    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.media.processor import MediaProcessor
    from cuteafd_b200.media.towers import AudioTower, AudioTowerConfig
    from cuteafd_b200.serve import api, tokenizer
    cfg = tiny_moe()
    tok = tokenizer.ByteTokenizer(cfg.vocab_size)
    ac = AudioTowerConfig(width=64, depth=1, heads=4, mlp=128, out_hidden=cfg.hidden)
    mp = MediaProcessor(cfg.vocab_size, cfg.hidden, None, AudioTower(ac, AudioTower.random_weights(ac)))
    L = signal(8000, 16, 21)
    flac, _ = encode([L], 8000, 16, [(4000, None, [{"kind": "fixed", "order": 2, "k": 9}], 7)] * 2)
    pcm = io.BytesIO()
    with wave.open(pcm, "wb") as w:
        w.setnchannels(1); w.setsampwidth(2); w.setframerate(8000)
        w.writeframes(struct.pack(f"<{len(L)}h", *L))

    def request(data, fmt):
        body = {"max_tokens": 2, "messages": [{"role": "user", "content": [
            {"type": "text", "text": "transcribe"}, {"type": "input_audio", "input_audio": {"data": base64.b64encode(data).decode(), "format": fmt}}]}]}
        return api.build_request(body, tok, cfg.vocab_size, media=mp)
    a, b = request(flac, "flac"), request(pcm.getvalue(), "wav")
    assert len(a.prompt) == len(b.prompt) and len(a.media) == len(b.media) == 1
    assert torch.equal(a.media[0].embeds, b.media[0].embeds) and a.media[0].key != b.media[0].key      # same rows, cached by content
    with pytest.raises(api.BadRequest, match="mp3"):
        request(b"ID3\x04" + bytes(200), "mp3")
