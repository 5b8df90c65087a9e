"""Audio input: WAV or FLAC bytes -> mono 16 kHz samples -> log-mel frames for the audio tower.

WAV (PCM 8 / 16 / 24 / 32-bit) through the standard library; FLAC through the C++ host runtime (``csrc/rt/flac.cc``:
every subframe type, both Rice codings, the stereo decorrelations, CRC-checked frames).  MP3 is refused by name.  A clip
is at most 300 s, a request at most 4 clips and 600 s (``MAX_CLIP_SECONDS``, ``MAX_CLIPS``, ``MAX_REQUEST_SECONDS``).

Counterparts: the reference's audio decode (hound / claxon / nanomp3; docs/multimodal-design.md:230 for the formats and
the limits) and its cuFFT mel front end (native/shared/cuda/audio_runtime.cu, pcm_audio_runtime.cu); here the transform
is ``torch.stft`` on whichever device the samples sit.
"""
from __future__ import annotations

import io
import math
import wave

import torch

from .image import MediaError

SAMPLE_RATE = 16000
N_FFT, HOP, N_MELS = 400, 160, 128
MAX_CLIP_SECONDS, MAX_REQUEST_SECONDS, MAX_CLIPS = 300, 600, 4


def decode_wav(raw: bytes) -> tuple[torch.Tensor, int]:
    """RIFF/WAVE bytes -> (float32 samples [n] in [-1, 1], mono; sample rate)."""
    try:
        with wave.open(io.BytesIO(raw)) as w:
            ch, width, rate, n = w.getnchannels(), w.getsampwidth(), w.getframerate(), w.getnframes()
            data = w.readframes(n)
    except (wave.Error, EOFError) as e:
        raise MediaError(f"cannot decode audio: {e}") from e
    if n > rate * MAX_CLIP_SECONDS:
        raise MediaError(f"audio clip longer than {MAX_CLIP_SECONDS} seconds")
    buf = bytearray(data)
    if width == 1:
        x = (torch.frombuffer(buf, dtype=torch.uint8).float() - 128.0) / 128.0
    elif width == 2:
        x = torch.frombuffer(buf, dtype=torch.int16).float() / 32768.0
    elif width == 3:
        b = torch.frombuffer(buf, dtype=torch.uint8).view(-1, 3).to(torch.int32)
        v = b[:, 0] | (b[:, 1] << 8) | (b[:, 2] << 16)
        x = torch.where(v >= 1 << 23, v - (1 << 24), v).float() / float(1 << 23)
    elif width == 4:
        x = torch.frombuffer(buf, dtype=torch.int32).float() / float(1 << 31)
    else:
        raise MediaError(f"unsupported sample width {width}")
    if ch > 1:
        x = x.view(-1, ch).mean(dim=1)
    return x.contiguous(), rate


def resample(x: torch.Tensor, rate: int, target: int = SAMPLE_RATE) -> torch.Tensor:
    if rate == target:
        return x
    try:
        import torchaudio.functional as AF
        return AF.resample(x, rate, target)
    except Exception:
        n = max(1, int(round(x.numel() * target / rate)))
        return torch.nn.functional.interpolate(x[None, None], size=n, mode="linear", align_corners=False)[0, 0]


def mel_filterbank(n_mels: int = N_MELS, n_fft: int = N_FFT, rate: int = SAMPLE_RATE) -> torch.Tensor:
    """Slaney-style triangular filters [n_mels, n_fft / 2 + 1]."""
    def hz_to_mel(f):
        return 2595.0 * math.log10(1.0 + f / 700.0)
    mels = torch.linspace(hz_to_mel(0.0), hz_to_mel(rate / 2), n_mels + 2)
    hz = 700.0 * (10.0 ** (mels / 2595.0) - 1.0)
    bins = torch.linspace(0, rate / 2, n_fft // 2 + 1)
    lo, ce, hi = hz[:-2, None], hz[1:-1, None], hz[2:, None]
    up, down = (bins[None] - lo) / (ce - lo), (hi - bins[None]) / (hi - ce)
    fb = torch.clamp(torch.minimum(up, down), min=0.0)
    return fb * (2.0 / (hi - lo))


def log_mel(samples: torch.Tensor) -> torch.Tensor:
    """float32 [n] at 16 kHz -> [frames, 128] log-mel, scaled to roughly [-1, 1] the way Whisper front ends do."""
    if samples.numel() < N_FFT:
        samples = torch.nn.functional.pad(samples, (0, N_FFT - samples.numel()))
    win = torch.hann_window(N_FFT, device=samples.device)
    spec = torch.stft(samples, N_FFT, HOP, window=win, return_complex=True)
    power = spec.abs().pow(2)[:, :-1]
    mel = mel_filterbank().to(samples.device) @ power
    lm = torch.clamp(mel, min=1e-10).log10()
    lm = torch.maximum(lm, lm.max() - 8.0)
    return ((lm + 4.0) / 4.0).T.contiguous()


_FLAC_ERRORS = {-1: "not a FLAC stream", -2: "no STREAMINFO block", -3: "truncated stream", -4: "bad frame header",
                -5: "checksum mismatch", -6: "bad subframe", -7: "bad residual coding", -8: "more samples than declared",
                -9: "sample size changes inside the stream"}


def decode_flac(raw: bytes) -> tuple[torch.Tensor, int]:
    """FLAC bytes -> (float32 samples [n] in [-1, 1], mono; sample rate)."""
    import ctypes as C

    from .._native import lib as native
    L = native.rt_lib()
    L.cafd_flac_info.argtypes = [C.c_char_p, C.c_uint64, C.POINTER(C.c_uint32), C.POINTER(C.c_int), C.POINTER(C.c_int), C.POINTER(C.c_uint64)]
    L.cafd_flac_decode_mono.argtypes, L.cafd_flac_decode_mono.restype = [C.c_char_p, C.c_uint64, C.c_void_p, C.c_uint64], C.c_longlong
    rate, ch, bits, total = C.c_uint32(), C.c_int(), C.c_int(), C.c_uint64()
    rc = L.cafd_flac_info(raw, len(raw), rate, ch, bits, total)
    if rc:
        raise MediaError(f"cannot decode audio: {_FLAC_ERRORS.get(rc, rc)}")
    limit = rate.value * MAX_CLIP_SECONDS
    if total.value > limit:
        raise MediaError(f"audio clip longer than {MAX_CLIP_SECONDS} seconds")
    def fail(code):
        if code == -8:                                       # more frames than the bound it was given
            return MediaError(f"audio clip longer than {MAX_CLIP_SECONDS} seconds" if not total.value else
                              "cannot decode audio: more samples than declared")
        return MediaError(f"cannot decode audio: {_FLAC_ERRORS.get(code, code)}")
    # a stream that does not declare its length is counted first (same bound), so the buffer is never a guess
    n = total.value or L.cafd_flac_decode_mono(raw, len(raw), None, limit)
    if n < 0:
        raise fail(n)
    out = torch.empty(max(n, 1), dtype=torch.float32)
    n = L.cafd_flac_decode_mono(raw, len(raw), out.data_ptr(), n)
    if n < 0:
        raise fail(n)
    return out[:n].contiguous(), rate.value


def decode_audio(raw: bytes) -> tuple[torch.Tensor, int]:
    """Container sniffed from the first bytes (the request's ``format`` field is a hint clients get wrong)."""
    if raw[:4] == b"RIFF":
        return decode_wav(raw)
    if raw[:4] == b"fLaC":
        return decode_flac(raw)
    if raw[:3] == b"ID3" or (len(raw) > 1 and raw[0] == 0xFF and raw[1] & 0xE0 == 0xE0):
        raise MediaError("mp3 audio is not decoded here: send wav or flac")
    raise MediaError("cannot decode audio: neither a WAV nor a FLAC stream")


def preprocess_audio(raw: bytes) -> torch.Tensor:
    x, rate = decode_audio(raw)
    return log_mel(resample(x, rate))
