"""Checkpoint number formats: encode / decode in plain PyTorch (CPU or GPU tensors).

These are the oracles for the dequantising kernels and the writers used to produce random-init
snapshots "as shipped".  Storage conventions follow the reference's loader
(rust/crates/cuteafd-loader/src/formats/fp8_experts.rs:1-33, plan/format.rs:29-135):

* FP8 block-128: E4M3 values, one fp32 scale per 128x128 weight block, multiply direction even
  when the tensor is named ``weight_scale_inv``; activations per row x 128-wide K block, amax/448
  (native/shared/cuda/fp8_gemv.cu:17-22).
* MXFP4: E2M1 two per byte (even element in the low nibble), one UE8M0 exponent per 32 along K.
* NVFP4: E2M1 as above, one E4M3 scale per 16 along K, one fp32 global scale (``weight_scale_2``,
  multiplier in the ModelOpt convention) (python/reference/cuteafd_reference/quant_ref.py:110-159).
* EXL3: 16-bit tail-biting trellis over 16x16 tiles, multiplicative-congruential codebook, H128
  Hadamard rotations with sign-scale vectors (python/tools/lib/exl3_reference.py:13-84).
"""
from __future__ import annotations

import math

import torch

E4M3_MAX = 448.0
E2M1_VALUES = torch.tensor([0.0, 0.5, 1.0, 1.5, 2.0, 3.0, 4.0, 6.0], dtype=torch.float32)
E2M1_MAX = 6.0
EXL3_MCG = 0xCBAC1FED


# ---- E4M3 ---------------------------------------------------------------------------------------------
def to_e4m3(x: torch.Tensor) -> torch.Tensor:
    return x.float().clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)


def fp8_quant_block128(w: torch.Tensor, block: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (E4M3 [N, K], fp32 scales [ceil(N/128), ceil(K/128)]); w ~= q * scale."""
    N, K = w.shape
    nb, kb = (N + block - 1) // block, (K + block - 1) // block
    pad = torch.zeros(nb * block, kb * block, dtype=torch.float32, device=w.device)
    pad[:N, :K] = w.float()
    blocks = pad.view(nb, block, kb, block)
    amax = blocks.abs().amax(dim=(1, 3))
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    q = to_e4m3(blocks / scale[:, None, :, None]).view(nb * block, kb * block)[:N, :K].contiguous()
    return q, scale.contiguous()


def fp8_dequant_block128(q: torch.Tensor, scale: torch.Tensor, block: int = 128) -> torch.Tensor:
    N, K = q.shape
    s = scale.repeat_interleave(block, 0)[:N].repeat_interleave(block, 1)[:, :K]
    return q.float() * s


def fp8_quant_rows(x: torch.Tensor, group: int = 128) -> tuple[torch.Tensor, torch.Tensor]:
    """Activations [T, K] -> (E4M3 [T, K], fp32 scales [T, K/group]), scale = amax/448 (1 if zero)."""
    T, K = x.shape
    assert K % group == 0
    g = x.float().view(T, K // group, group)
    amax = g.abs().amax(-1)
    scale = torch.where(amax > 0, amax / E4M3_MAX, torch.ones_like(amax))
    return to_e4m3(g / scale[..., None]).view(T, K), scale.contiguous()


def fp8_dequant_rows(q: torch.Tensor, scale: torch.Tensor, group: int = 128) -> torch.Tensor:
    T, K = q.shape
    return (q.float().view(T, K // group, group) * scale[..., None]).view(T, K)


# ---- E2M1 helpers --------------------------------------------------------------------------------------
def _e2m1_encode(x: torch.Tensor) -> torch.Tensor:
    """Nearest E2M1 code (ties to the even code), sign in bit 3; x already divided by its scale."""
    mag = x.abs().clamp(max=E2M1_MAX)
    vals = E2M1_VALUES.to(x.device)
    d = (mag[..., None] - vals).abs()
    # ties -> even code index: bias the odd codes by a hair
    d = d + (torch.arange(8, device=x.device) % 2).float() * 1e-7
    code = d.argmin(-1).to(torch.uint8)
    neg = (x < 0) & (code != 0)
    return code | (neg.to(torch.uint8) << 3)


def _e2m1_decode(code: torch.Tensor) -> torch.Tensor:
    vals = E2M1_VALUES.to(code.device)
    mag = vals[(code & 7).long()]
    return torch.where((code & 8) != 0, -mag, mag)


def pack_nibbles(codes: torch.Tensor) -> torch.Tensor:
    """[..., K] 4-bit codes -> [..., K/2] bytes, even element in the low nibble."""
    return (codes[..., 0::2] & 0xF) | ((codes[..., 1::2] & 0xF) << 4)


def unpack_nibbles(packed: torch.Tensor) -> torch.Tensor:
    out = torch.empty(*packed.shape[:-1], packed.shape[-1] * 2, dtype=torch.uint8, device=packed.device)
    out[..., 0::2] = packed & 0xF
    out[..., 1::2] = (packed >> 4) & 0xF
    return out


# ---- MXFP4: E2M1 + UE8M0 per 32 ------------------------------------------------------------------------
def mxfp4_quant(w: torch.Tensor, group: int = 32) -> tuple[torch.Tensor, torch.Tensor]:
    """[N, K] -> (packed uint8 [N, K/2], UE8M0 uint8 [N, K/group]); scale = 2^(e-127)."""
    N, K = w.shape
    g = w.float().view(N, K // group, group)
    amax = g.abs().amax(-1).clamp_min(2.0 ** -126)
    e = torch.ceil(torch.log2(amax / E2M1_MAX)).clamp(-127, 127)
    scale = torch.exp2(e)
    codes = _e2m1_encode(g / scale[..., None]).view(N, K)
    return pack_nibbles(codes), (e + 127).to(torch.uint8)


def mxfp4_dequant(packed: torch.Tensor, ue8m0: torch.Tensor, group: int = 32) -> torch.Tensor:
    vals = _e2m1_decode(unpack_nibbles(packed))
    N, K = vals.shape
    scale = torch.exp2(ue8m0.float() - 127.0)
    return (vals.view(N, K // group, group) * scale[..., None]).view(N, K)


# ---- NVFP4: E2M1 + E4M3 per 16 + fp32 global -----------------------------------------------------------
def nvfp4_quant(w: torch.Tensor, group: int = 16) -> tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[N, K] -> (packed uint8 [N, K/2], E4M3 block scales [N, K/16], fp32 global scale).

    w ~= e2m1 * block_scale * global; global = amax / (448 * 6) so block scales fit E4M3."""
    N, K = w.shape
    wf = w.float()
    amax = wf.abs().max().clamp_min(1e-12)
    glob = amax / (E4M3_MAX * E2M1_MAX)
    g = wf.view(N, K // group, group)
    bs = to_e4m3(g.abs().amax(-1) / E2M1_MAX / glob)
    eff = bs.float() * glob
    safe = torch.where(eff > 0, eff, torch.ones_like(eff))
    codes = _e2m1_encode(g / safe[..., None]).view(N, K)
    return pack_nibbles(codes), bs, glob.reshape(1).float()


def nvfp4_dequant(packed: torch.Tensor, block_scale: torch.Tensor, global_scale: torch.Tensor, group: int = 16) -> torch.Tensor:
    vals = _e2m1_decode(unpack_nibbles(packed))
    N, K = vals.shape
    s = block_scale.float() * global_scale.float()
    return (vals.view(N, K // group, group) * s[..., None]).view(N, K)


# ---- EXL3 trellis ----------------------------------------------------------------------------------------
def _exl3_lane_permutation() -> torch.Tensor:
    perm = []
    for lane in range(32):
        row, col = (lane % 4) * 2, lane // 4
        for dr, dc in ((0, 0), (1, 0), (8, 0), (9, 0), (0, 8), (1, 8), (8, 8), (9, 8)):
            perm.append((row + dr) * 16 + col + dc)
    return torch.tensor(perm, dtype=torch.long)


def exl3_decode_inner(trellis: torch.Tensor) -> torch.Tensor:
    """int16 [K/16, N/16, 16*bits] -> float32 [K, N] (before the Hadamard rotations)."""
    Kt, Nt, W = trellis.shape
    bits = W // 16
    assert W == 16 * bits and 1 <= bits <= 8
    words = (trellis.to(torch.int32) & 0xFFFF).view(Kt, Nt, W // 2, 2).flip(-1).reshape(Kt, Nt, W)
    # bit stream of 16*bits*16 bits, MSB first inside each (swapped) word; 256 symbols of `bits` bits
    shifts = torch.arange(15, -1, -1, device=trellis.device)
    stream = ((words[..., None] >> shifts) & 1).reshape(Kt, Nt, W * 16)
    weights = (1 << torch.arange(bits - 1, -1, -1, device=trellis.device))
    # segment s = words [s*bits, (s+1)*bits): sixteen `bits`-wide symbols, MSB first; symbol index
    # inside the tile is segment * 16 + position
    symbols = (stream.view(Kt, Nt, 16, 16, bits) * weights).sum(-1).reshape(Kt, Nt, 256)
    hist = (16 + bits - 1) // bits - 1
    state = torch.zeros(Kt, Nt, dtype=torch.int64, device=trellis.device)
    for p in range(256 - hist, 256):
        state = ((state << bits) | symbols[..., p]) & 0xFFFF
    codes = torch.empty(Kt, Nt, 256, dtype=torch.int64, device=trellis.device)
    for p in range(256):
        state = ((state << bits) | symbols[..., p]) & 0xFFFF
        codes[..., p] = state
    raw = (codes * EXL3_MCG) & 0xFFFFFFFF
    raw = 0x3B603B60 ^ (raw & 0x8FFF8FFF)
    lo = (raw & 0xFFFF).to(torch.int32).to(torch.int16).view(torch.float16).float()
    hi = ((raw >> 16) & 0xFFFF).to(torch.int32).to(torch.int16).view(torch.float16).float()
    dec = lo + hi
    inv = torch.argsort(_exl3_lane_permutation()).to(trellis.device)
    dec = dec[..., inv]
    return dec.view(Kt, Nt, 16, 16).permute(0, 2, 1, 3).reshape(Kt * 16, Nt * 16)


def hadamard128(x: torch.Tensor) -> torch.Tensor:
    """Normalised block Hadamard transform over groups of 128 along the last dimension."""
    shape = x.shape
    assert shape[-1] % 128 == 0
    v = x.double().reshape(-1, 128).clone()
    step = 1
    while step < 128:
        p = v.view(-1, 128 // (2 * step), 2, step)
        a, b = p[:, :, 0].clone(), p[:, :, 1].clone()
        p[:, :, 0], p[:, :, 1] = a + b, a - b
        step *= 2
    return (v / math.sqrt(128.0)).view(shape)


def exl3_dequant(trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor) -> torch.Tensor:
    """Effective weight [K, N] (input dim first) as float64."""
    inner = exl3_decode_inner(trellis).double()
    w = hadamard128(inner.T).T * suh.double()[:, None]
    return hadamard128(w) * svh.double()[None, :]


def exl3_random(K: int, N: int, bits: int, gen: torch.Generator, scale: float = 0.02):
    """Random EXL3 tensors of a given geometry (any bit pattern is a valid trellis)."""
    trellis = torch.randint(-32768, 32768, (K // 16, N // 16, 16 * bits), generator=gen, dtype=torch.int32).to(torch.int16)
    suh = (torch.randint(0, 2, (K,), generator=gen).float() * 2 - 1).to(torch.float16)
    svh = ((torch.randint(0, 2, (N,), generator=gen).float() * 2 - 1) * scale).to(torch.float16)
    return trellis, suh, svh
