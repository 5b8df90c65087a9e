"""EXL3 encoder: trellis-coded quantisation of a weight matrix into the tensors ``exl3_dequant`` reads.

The stored form is the inverse of the decoder in ``quant/codecs.py``:

    W[K, N] = diag(suh) . H_K . inner . H_N . diag(svh)        (H = normalised 128-block Hadamard, H.H = I)

so the encoder rotates ``inner_target = H_K . diag(1/suh) . W . diag(1/svh) . H_N`` with random signs (which makes
the entries close to Gaussian), scales every output column to the codebook's spread, and searches, for every
16 x 16 tile, the 256-symbol bit stream whose decoded values are closest to the tile.  A symbol of ``bits`` bits
shifts into a 16-bit window and the window indexes the computed codebook, so the search is a Viterbi pass over
65 536 states with 2**bits predecessors per state; the stream is circular (the decoder pre-rolls the window with the
last symbols), which the search meets with the usual two passes: a free pass fixes the window at the middle of the
tile, a second pass starts and ends in that window.

Plain rounding in the rotated space is used (no calibration Hessian); ``proxy_error`` reports the relative error.
Counterpart: the reference's EXL3 quantiser (python/cuteafd_runtime/exl3_quantizer.py) and its trellis decoder
(native/shared/cuda/exl3_codebook.cuh); the codebook arithmetic is shared with ``codecs.exl3_decode_inner``.
"""
from __future__ import annotations

import torch

from . import codecs

_STATES = 1 << 16


def codebook(device: str | torch.device = "cpu") -> torch.Tensor:
    """Decoded value of every 16-bit window (float32 [65536])."""
    s = torch.arange(_STATES, dtype=torch.int64, device=device)
    raw = (s * codecs.EXL3_MCG) & 0xFFFFFFFF
    raw = 0x3B603B60 ^ (raw & 0x8FFF8FFF)
    lo = (raw & 0xFFFF).to(torch.int32).to(torch.int16).view(torch.float16).float()
    hi = ((raw >> 16) & 0xFFFF).to(torch.int32).to(torch.int16).view(torch.float16).float()
    return lo + hi


def _viterbi(target: torch.Tensor, cb: torch.Tensor, bits: int, start: torch.Tensor | None, order: torch.Tensor):
    """One pass over the positions in ``order``.  target [tiles, 256] (stream order).

    start None: every window may open the path.  start [tiles]: the path opens in that window (the window before the
    first position of ``order``) and must close in it.  Returns (window after every position [tiles, 256] indexed by
    stream position, total cost [tiles])."""
    tiles = target.shape[0]
    dev = target.device
    low = _STATES >> bits                       # windows that share their low 16-bits bits share predecessors
    if start is None:
        cost = torch.zeros(tiles, _STATES, device=dev)
    else:
        cost = torch.full((tiles, _STATES), float("inf"), device=dev)
        cost.scatter_(1, start[:, None], 0.0)
    back = torch.empty(order.numel(), tiles, low, dtype=torch.uint8, device=dev)
    for step, p in enumerate(order.tolist()):
        # predecessor of window n: (top << (16 - bits)) | (n >> bits) for any top
        m, arg = cost.view(tiles, 1 << bits, low).min(dim=1)
        back[step] = arg.to(torch.uint8)
        err = (cb[None, :] - target[:, p, None]) ** 2
        cost = m.repeat_interleave(1 << bits, dim=1) + err
    if start is None:
        total, end = cost.min(dim=1)
    else:
        end = start
        total = cost.gather(1, start[:, None])[:, 0]
    windows = torch.empty(tiles, 256, dtype=torch.int64, device=dev)
    rows = torch.arange(tiles, device=dev)
    state = end
    for step in range(order.numel() - 1, -1, -1):
        windows[:, order[step]] = state
        top = back[step][rows, state >> bits].to(torch.int64)
        state = (top << (16 - bits)) | (state >> bits)
    return windows, total


def encode_tiles(target: torch.Tensor, bits: int) -> tuple[torch.Tensor, torch.Tensor]:
    """target [tiles, 256] in stream order -> (symbols [tiles, 256] int64, squared error [tiles])."""
    cb = codebook(target.device)
    fwd = torch.arange(256)
    free, _ = _viterbi(target, cb, bits, None, fwd)
    mid = free[:, 127]                                            # window after position 127 = before position 128
    rot = torch.cat([torch.arange(128, 256), torch.arange(0, 128)])
    windows, total = _viterbi(target, cb, bits, mid, rot)
    return windows & ((1 << bits) - 1), total


def _pack(symbols: torch.Tensor, bits: int) -> torch.Tensor:
    """symbols [tiles, 256] -> int16 words [tiles, 16 * bits] in the stored (pair-swapped) order."""
    tiles = symbols.shape[0]
    shifts = torch.arange(bits - 1, -1, -1, device=symbols.device)
    stream = ((symbols[..., None] >> shifts) & 1).reshape(tiles, 16 * bits, 16)       # 16-bit words, MSB first
    weights = (1 << torch.arange(15, -1, -1, device=symbols.device))
    words = (stream * weights).sum(-1)
    words = words.view(tiles, 8 * bits, 2).flip(-1).reshape(tiles, 16 * bits)
    return torch.where(words >= 32768, words - 65536, words).to(torch.int16)


def exl3_quantize(w: torch.Tensor, bits: int, gen: torch.Generator | None = None, tile_batch: int = 128,
                  device: str | torch.device | None = None) -> dict[str, torch.Tensor]:
    """w [K, N] (input dimension first, both multiples of 128) -> {"trellis", "suh", "svh", "proxy_error"}."""
    K, N = w.shape
    assert K % 128 == 0 and N % 128 == 0 and 1 <= bits <= 8
    gen = gen or torch.Generator().manual_seed(0)
    dev = torch.device(device) if device is not None else w.device
    wd = w.double().cpu()
    su = (torch.randint(0, 2, (K,), generator=gen).double() * 2 - 1)
    sv = (torch.randint(0, 2, (N,), generator=gen).double() * 2 - 1)
    a = codecs.hadamard128((wd * su[:, None]).T.contiguous()).T.contiguous()          # H_K . diag(1/su) . W  (su = +-1)
    cb = codebook("cpu").double()
    cb_rms = cb.pow(2).mean().sqrt()
    col = a.pow(2).mean(dim=0).sqrt().clamp_min(1e-12) / cb_rms
    svh = (sv * col).to(torch.float16)
    suh = su.to(torch.float16)
    inner_t = codecs.hadamard128((a / svh.double()[None, :]).contiguous())            # ... . diag(1/svh) . H_N
    # tiles in stream order
    Kt, Nt = K // 16, N // 16
    tiles = inner_t.view(Kt, 16, Nt, 16).permute(0, 2, 1, 3).reshape(Kt * Nt, 256)
    perm = codecs._exl3_lane_permutation()
    stream_t = tiles[:, perm].float().to(dev)
    sym = torch.empty(Kt * Nt, 256, dtype=torch.int64, device=dev)
    for t0 in range(0, Kt * Nt, tile_batch):
        s, _ = encode_tiles(stream_t[t0 : t0 + tile_batch], bits)
        sym[t0 : t0 + tile_batch] = s
    trellis = _pack(sym, bits).view(Kt, Nt, 16 * bits).cpu()
    got = codecs.exl3_dequant(trellis, suh, svh)
    err = ((got - wd).pow(2).sum() / wd.pow(2).sum().clamp_min(1e-30)).sqrt()
    return {"trellis": trellis, "suh": suh, "svh": svh, "proxy_error": err.float()}
