"""From chat content parts to what the engines consume: placeholder tokens in the prompt and the embedding rows that
replace them.

An image or audio clip becomes ``<start> pad x n <end>`` in the token stream, where n is the number of rows its tower
produces.  The pad positions do not carry the tokenizer's pad id but a pseudo id above the vocabulary, derived from
the content hash: the prefix cache (which chains hashes of token ids) then tells two different images apart with no
extra key, and the engines recognise override rows as "id >= vocab_size".  ``MediaSpan`` carries the rows.

Counterparts: media keys in the prefix cache and the placeholder expansion of rust/crates/cuteafd-api/src/openai/
media*.rs and rust/crates/cuteafd-engine/src/media/.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from . import audio as A
from . import image as I
from .cache import EmbeddingCache


@dataclass
class MediaSpan:
    start: int                 # prompt position of the first overridden row
    embeds: torch.Tensor       # [length, hidden]
    key: bytes
    kind: str

    @property
    def length(self) -> int:
        return self.embeds.shape[0]


def pseudo_id(key: bytes, vocab_size: int) -> int:
    """Token id that stands for "row of media item ``key``": above the vocabulary, inside int32."""
    span = (1 << 31) - 1 - vocab_size - 1
    return vocab_size + 1 + int.from_bytes(key[:8], "little") % span


def overrides_for(spans: list[MediaSpan], start: int, n: int) -> tuple[list[int], torch.Tensor] | None:
    """Rows (relative to ``start``) and their embeddings for the prompt window [start, start + n)."""
    rows, vals = [], []
    for s in spans or ():
        lo, hi = max(start, s.start), min(start + n, s.start + s.length)
        if lo < hi:
            rows += list(range(lo - start, hi - start))
            vals.append(s.embeds[lo - s.start: hi - s.start])
    if not rows:
        return None
    return rows, torch.cat(vals, dim=0)


class MediaProcessor:
    """Owns the towers and the embedding cache of one serving process."""

    def __init__(self, vocab_size: int, hidden: int, vision=None, audio=None, cache: EmbeddingCache | None = None,
                 start_id: int | None = None, end_id: int | None = None, max_items: int = 16):
        self.vocab_size, self.hidden = vocab_size, hidden
        self.vision, self.audio = vision, audio
        self.cache = cache or EmbeddingCache()
        self.start_id, self.end_id = start_id, end_id
        self.max_items = max_items
        self.encoded = 0
        self._seconds: dict[bytes, float] = {}            # clip length by content key (for the per-request bound)

    # ---- one item ----------------------------------------------------------------------------------------
    def encode_image(self, raw: bytes) -> tuple[bytes, torch.Tensor]:
        if self.vision is None:
            raise I.MediaError("this deployment serves no vision tower")
        key = I.content_key(raw, "image")
        hit = self.cache.get(key)
        if hit is not None:
            return key, hit
        cfg = self.vision.cfg
        patches, grid = I.preprocess_image(I.decode_image(raw), cfg.patch, cfg.merge)
        out = self.vision.forward(patches, grid)
        assert out.shape == (self.vision.rows_for(grid), self.hidden)
        self.cache.put(key, out)
        self.encoded += 1
        return key, out

    def encode_audio(self, raw: bytes) -> tuple[bytes, torch.Tensor]:
        if self.audio is None:
            raise I.MediaError("this deployment serves no audio tower")
        key = I.content_key(raw, "audio")
        hit = self.cache.get(key)
        if hit is not None:
            return key, hit
        x, rate = A.decode_audio(raw)
        self._seconds[key] = x.numel() / rate
        out = self.audio.forward(A.log_mel(A.resample(x, rate)))
        self.cache.put(key, out)
        self.encoded += 1
        return key, out

    def audio_seconds(self, raw: bytes) -> float:
        """Length of a clip that has been encoded (remembered by content, so a cached clip is not decoded again)."""
        key = I.content_key(raw, "audio")
        if key not in self._seconds:
            x, rate = A.decode_audio(raw)
            self._seconds[key] = x.numel() / rate
            while len(self._seconds) > 4096:
                self._seconds.pop(next(iter(self._seconds)))
        return self._seconds[key]

    # ---- a whole conversation ------------------------------------------------------------------------------
    def expand(self, segments: list, encode_text) -> tuple[list[int], list[MediaSpan]]:
        """``segments``: strings and ("image" | "audio", bytes) pairs in prompt order.  ``encode_text(str) -> ids``.
        Returns the prompt ids (pseudo ids at media rows) and the spans."""
        ids: list[int] = []
        spans: list[MediaSpan] = []
        clips, frames = 0, 0
        for seg in segments:
            if isinstance(seg, str):
                if seg:
                    ids += encode_text(seg)
                continue
            kind, raw = seg
            if len(spans) >= self.max_items:
                raise I.MediaError(f"more than {self.max_items} media items in one request")
            key, emb = self.encode_image(raw) if kind == "image" else self.encode_audio(raw)
            if kind == "audio":                               # per-request bounds: clips, and their summed length
                clips, frames = clips + 1, frames + self.audio_seconds(raw)
                if clips > A.MAX_CLIPS:
                    raise I.MediaError(f"more than {A.MAX_CLIPS} audio clips in one request")
                if frames > A.MAX_REQUEST_SECONDS:
                    raise I.MediaError(f"more than {A.MAX_REQUEST_SECONDS} seconds of audio in one request")
            if self.start_id is not None:
                ids.append(self.start_id)
            spans.append(MediaSpan(len(ids), emb, key, kind))
            ids += [pseudo_id(key, self.vocab_size)] * emb.shape[0]
            if self.end_id is not None:
                ids.append(self.end_id)
        return ids, spans

    def describe(self) -> dict:
        return {"vision": self.vision is not None, "audio": self.audio is not None, "encoded": self.encoded,
                "cache": self.cache.describe()}
