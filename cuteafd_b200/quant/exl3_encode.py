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

Without calibration data the tiles are rounded independently in the rotated space; with the input Hessian of the layer
(``hessian=``) the 16-row blocks are encoded in sequence with GPTQ-style error feedback, which cuts the output error
the calibration inputs see several times over.  ``proxy_error`` reports the relative weight error.
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


def _rotate_hessian(h: torch.Tensor, su: torch.Tensor) -> torch.Tensor:
    """Hessian of the layer input x -> Hessian of the rotated input x' = H_K (x * su)."""
    d = h.double() * su[:, None] * su[None, :]
    d = codecs.hadamard128(d.contiguous())                      # columns
    return codecs.hadamard128(d.T.contiguous()).T.contiguous()   # rows


def exl3_quantize(w: torch.Tensor, bits: int, gen: torch.Generator | None = None, tile_batch: int = 128,
                  device: str | torch.device | None = None, hessian: torch.Tensor | None = None,
                  damp: float = 0.01) -> dict[str, torch.Tensor]:
    """w [K, N] (input dimension first, both multiples of 128) -> {"trellis", "suh", "svh", "proxy_error"}.

    ``hessian`` [K, K] (sum of x x^T over calibration inputs) switches from plain rounding to block error feedback:
    the 16-row blocks of the rotated weight are encoded one after the other, and the error of a block is spread over
    the rows still to come through the inverse Hessian's Cholesky factor (the GPTQ update with the trellis as the
    block quantiser), which lowers the output error tr(E^T H E) the calibration data sees.  ``hessian_error`` in the
    result is that quantity relative to tr(W^T H W)."""
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
    Kt, Nt = K // 16, N // 16
    perm = codecs._exl3_lane_permutation()

    def encode_rows(block: torch.Tensor) -> torch.Tensor:
        """[16 * r, N] rows of the rotated weight -> int16 words [r, Nt, 16 * bits]."""
        r = block.shape[0] // 16
        tiles = block.view(r, 16, Nt, 16).permute(0, 2, 1, 3).reshape(r * Nt, 256)
        stream_t = tiles[:, perm].float().to(dev)
        sym = torch.empty(r * Nt, 256, dtype=torch.int64, device=dev)
        for t0 in range(0, r * Nt, tile_batch):
            sym[t0:t0 + tile_batch] = encode_tiles(stream_t[t0:t0 + tile_batch], bits)[0]
        return _pack(sym, bits).view(r, Nt, 16 * bits).cpu()

    out: dict[str, torch.Tensor] = {}
    if hessian is None:
        trellis = encode_rows(inner_t)
    else:
        assert hessian.shape == (K, K)
        hr = _rotate_hessian(hessian.cpu(), su)
        hr = hr + damp * hr.diagonal().mean() * torch.eye(K, dtype=torch.float64)
        hinv = torch.linalg.cholesky(torch.linalg.inv(hr), upper=True)               # [K, K]
        wt = inner_t.T.clone()                                                       # [N, K]: columns = input rows
        trellis = torch.empty(Kt, Nt, 16 * bits, dtype=torch.int16)
        for kb in range(Kt):
            blk = slice(16 * kb, 16 * kb + 16)
            words = encode_rows(wt[:, blk].T.contiguous())
            trellis[kb] = words[0]
            q = codecs.exl3_decode_inner(words).double()                              # [16, N]
            err = (wt[:, blk] - q.T) @ torch.linalg.inv(hinv[blk, blk])
            if kb + 1 < Kt:
                wt[:, 16 * kb + 16:] -= err @ hinv[blk, 16 * kb + 16:]
        e = codecs.exl3_decode_inner(trellis).double() - inner_t
        out["hessian_error"] = (torch.einsum("kn,kj,jn->", e, _rotate_hessian(hessian.cpu(), su), e)
                                / torch.einsum("kn,kj,jn->", inner_t, _rotate_hessian(hessian.cpu(), su), inner_t).clamp_min(1e-30)).float()
    got = codecs.exl3_dequant(trellis, suh, svh)
    err = ((got - wd).pow(2).sum() / wd.pow(2).sum().clamp_min(1e-30)).sqrt()
    out.update({"trellis": trellis, "suh": suh, "svh": svh, "proxy_error": err.float()})
    return out


def hessian_error(w: torch.Tensor, q: dict, hessian: torch.Tensor) -> float:
    """tr(E^T H E) / tr(W^T H W) for a quantised result ``q`` of ``w`` [K, N] under the input Hessian ``hessian``."""
    e = codecs.exl3_dequant(q["trellis"], q["suh"], q["svh"]) - w.double()
    h = hessian.double()
    return float(torch.einsum("kn,kj,jn->", e, h, e) / torch.einsum("kn,kj,jn->", w.double(), h, w.double()).clamp_min(1e-30))
