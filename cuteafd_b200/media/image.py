"""Image input: bytes -> RGB pixels -> patch rows for the vision tower.

The resize rule keeps the aspect ratio, makes both sides multiples of ``patch * merge`` (the tower merges
``merge x merge`` patches into one language-model row) and keeps the pixel count inside a budget, as the bundled
vision families do.  Only ``data:`` URLs and raw bytes are accepted: the serving process fetches nothing.

Counterparts: rust/crates/cuteafd-loader/src/media/ (decode + preprocess), rust/crates/cuteafd-api/src/openai/media*.rs.
"""
from __future__ import annotations

import base64
import hashlib
import io
import math

import torch

CLIP_MEAN = (0.48145466, 0.4578275, 0.40821073)
CLIP_STD = (0.26862954, 0.26130258, 0.27577711)
MAX_IMAGE_BYTES = 32 << 20


class MediaError(ValueError):
    pass


def bytes_from_url(url: str) -> bytes:
    """``data:<mime>;base64,<payload>`` only."""
    if not isinstance(url, str) or not url.startswith("data:"):
        raise MediaError("only data: URLs are served (the server fetches no remote media)")
    head, _, payload = url.partition(",")
    if not payload:
        raise MediaError("empty data URL")
    try:
        raw = base64.b64decode(payload, validate=False) if head.endswith(";base64") else payload.encode()
    except Exception as e:
        raise MediaError(f"invalid base64 payload: {e}") from e
    if len(raw) > MAX_IMAGE_BYTES:
        raise MediaError("media payload too large")
    return raw


def content_key(raw: bytes, kind: str = "image") -> bytes:
    return hashlib.blake2b(kind.encode() + b"\0" + raw, digest_size=16).digest()


def decode_image(raw: bytes) -> torch.Tensor:
    """PNG / JPEG / WebP / BMP / GIF (first frame) bytes -> uint8 [H, W, 3]."""
    from PIL import Image
    try:
        im = Image.open(io.BytesIO(raw))
        im = im.convert("RGB")
    except Exception as e:
        raise MediaError(f"cannot decode image: {e}") from e
    if im.width * im.height > 64_000_000:
        raise MediaError("image too large")
    return torch.frombuffer(bytearray(im.tobytes()), dtype=torch.uint8).view(im.height, im.width, 3)


def smart_resize(h: int, w: int, factor: int = 28, min_pixels: int = 56 * 56, max_pixels: int = 1280 * 28 * 28) -> tuple[int, int]:
    if min(h, w) <= 0:
        raise MediaError("empty image")
    if max(h, w) / min(h, w) > 200:
        raise MediaError("aspect ratio beyond 200:1")
    nh, nw = max(factor, round(h / factor) * factor), max(factor, round(w / factor) * factor)
    if nh * nw > max_pixels:
        beta = math.sqrt(h * w / max_pixels)
        nh, nw = max(factor, math.floor(h / beta / factor) * factor), max(factor, math.floor(w / beta / factor) * factor)
    elif nh * nw < min_pixels:
        beta = math.sqrt(min_pixels / (h * w))
        nh, nw = math.ceil(h * beta / factor) * factor, math.ceil(w * beta / factor) * factor
    return nh, nw


def preprocess_image(pixels: torch.Tensor, patch: int = 14, merge: int = 2, min_pixels: int = 56 * 56,
                     max_pixels: int = 1280 * 28 * 28) -> tuple[torch.Tensor, tuple[int, int]]:
    """uint8 [H, W, 3] -> (patch rows [gh * gw, 3 * patch * patch] fp32, (gh, gw)).

    Rows are ordered so that the ``merge x merge`` patches of one merged cell are consecutive (cell-major), which lets
    the tower's merger be a reshape."""
    h, w, _ = pixels.shape
    nh, nw = smart_resize(h, w, patch * merge, min_pixels, max_pixels)
    x = pixels.permute(2, 0, 1).float()[None] / 255.0
    x = torch.nn.functional.interpolate(x, size=(nh, nw), mode="bicubic", align_corners=False, antialias=True).clamp_(0, 1)[0]
    mean, std = torch.tensor(CLIP_MEAN)[:, None, None], torch.tensor(CLIP_STD)[:, None, None]
    x = (x - mean) / std
    gh, gw = nh // patch, nw // patch
    # [3, gh/m, m, p, gw/m, m, p] -> [gh/m, gw/m, m, m, 3, p, p]
    x = x.view(3, gh // merge, merge, patch, gw // merge, merge, patch).permute(1, 4, 2, 5, 0, 3, 6)
    return x.reshape(gh * gw, 3 * patch * patch).contiguous(), (gh, gw)


def patch_positions(gh: int, gw: int, merge: int = 2) -> torch.Tensor:
    """(row, column) of every patch in the cell-major order of ``preprocess_image`` -> int64 [gh * gw, 2]."""
    r = torch.arange(gh).view(gh // merge, 1, merge, 1).expand(gh // merge, gw // merge, merge, merge)
    c = torch.arange(gw).view(1, gw // merge, 1, merge).expand(gh // merge, gw // merge, merge, merge)
    return torch.stack([r.reshape(-1), c.reshape(-1)], dim=1)
