"""Vision and audio towers: transformer encoders whose outputs are rows in the language model's hidden space.

Vision (the Qwen-VL / GLM-V pattern): linear patch embedding, pre-norm blocks with full (bidirectional) attention and
2-D rotary positions, GELU MLP, then a merger that concatenates each ``merge x merge`` cell and projects it to the
language model's width.  Audio (the Whisper pattern): two strided 1-D convolutions over log-mel frames, sinusoidal
positions, pre-norm blocks, average pooling by two, projection.

On a GPU the projections run on this package's tcgen05 GEMM (``ops.kernels.linear``) in bf16; attention inside the
towers is PyTorch's scaled-dot-product attention (a library kernel: the towers are a few percent of a request and not
on the decode path).  On the CPU everything is fp32 PyTorch, which is also the oracle the GPU path is tested against.

Counterparts: native/shared/cuda/vision*.cu(h) (CUDA towers + cuBLAS), audio_runtime.cu, and the encoder placement
logic in rust/crates/cuteafd-daemon/src/shared/vision*.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch
import torch.nn.functional as F

from .image import patch_positions


@dataclass(frozen=True)
class VisionTowerConfig:
    patch: int = 14
    merge: int = 2
    width: int = 1280
    depth: int = 32
    heads: int = 16
    mlp: int = 5120
    out_hidden: int = 2048
    eps: float = 1e-6

    @property
    def patch_dim(self) -> int:
        return 3 * self.patch * self.patch


@dataclass(frozen=True)
class AudioTowerConfig:
    mels: int = 128
    width: int = 1280
    depth: int = 32
    heads: int = 20
    mlp: int = 5120
    out_hidden: int = 2048
    eps: float = 1e-5


def _linear(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor | None) -> torch.Tensor:
    """x [n, K] @ w[N, K].T + b.  bf16 CUDA tensors with friendly shapes take the tcgen05 GEMM."""
    if x.is_cuda and x.dtype == torch.bfloat16 and x.shape[1] % 64 == 0 and w.shape[0] % 16 == 0 and x.shape[0] > 0:
        from ..ops import kernels as K
        y = K.linear(x.contiguous(), w)
        return y if b is None else y + b
    return F.linear(x, w, b)


def _rope_2d(pos: torch.Tensor, head_dim: int, theta: float = 10000.0) -> tuple[torch.Tensor, torch.Tensor]:
    """cos / sin [n, head_dim]: the first half of the rotary pairs turns with the row, the second with the column."""
    quarter = head_dim // 4
    inv = 1.0 / (theta ** (torch.arange(quarter, dtype=torch.float32, device=pos.device) / quarter))
    ang = torch.cat([pos[:, 0:1].float() * inv, pos[:, 1:2].float() * inv], dim=1)       # [n, head_dim / 2]
    ang = torch.cat([ang, ang], dim=1)
    return ang.cos(), ang.sin()


def _rotate_half(x: torch.Tensor) -> torch.Tensor:
    a, b = x.chunk(2, dim=-1)
    return torch.cat([-b, a], dim=-1)


class _Encoder:
    """Shared transformer trunk over a weight dictionary ``{name: tensor}``."""

    def __init__(self, weights: dict[str, torch.Tensor], depth: int, heads: int, eps: float):
        self.w, self.depth, self.heads, self.eps = weights, depth, heads, eps

    def block(self, i: int, x: torch.Tensor, rope: tuple[torch.Tensor, torch.Tensor] | None) -> torch.Tensor:
        w, p = self.w, f"blocks.{i}."
        n, d = x.shape
        hd = d // self.heads
        y = F.layer_norm(x, (d,), w[p + "norm1.weight"], w[p + "norm1.bias"], self.eps)
        qkv = _linear(y, w[p + "attn.qkv.weight"], w[p + "attn.qkv.bias"]).view(n, 3, self.heads, hd)
        q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
        if rope is not None:
            cos, sin = rope[0][:, None, :].to(q.dtype), rope[1][:, None, :].to(q.dtype)
            q, k = q * cos + _rotate_half(q) * sin, k * cos + _rotate_half(k) * sin
        o = F.scaled_dot_product_attention(q.transpose(0, 1)[None], k.transpose(0, 1)[None], v.transpose(0, 1)[None])[0]
        x = x + _linear(o.transpose(0, 1).reshape(n, d), w[p + "attn.proj.weight"], w[p + "attn.proj.bias"])
        y = F.layer_norm(x, (d,), w[p + "norm2.weight"], w[p + "norm2.bias"], self.eps)
        y = F.gelu(_linear(y, w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"]))
        return x + _linear(y, w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"])


def _init_blocks(w: dict, depth: int, width: int, mlp: int, gen: torch.Generator, std: float) -> None:
    def r(*shape):
        return torch.randn(*shape, generator=gen) * std
    for i in range(depth):
        p = f"blocks.{i}."
        w[p + "norm1.weight"], w[p + "norm1.bias"] = torch.ones(width), torch.zeros(width)
        w[p + "norm2.weight"], w[p + "norm2.bias"] = torch.ones(width), torch.zeros(width)
        w[p + "attn.qkv.weight"], w[p + "attn.qkv.bias"] = r(3 * width, width), torch.zeros(3 * width)
        w[p + "attn.proj.weight"], w[p + "attn.proj.bias"] = r(width, width), torch.zeros(width)
        w[p + "mlp.fc1.weight"], w[p + "mlp.fc1.bias"] = r(mlp, width), torch.zeros(mlp)
        w[p + "mlp.fc2.weight"], w[p + "mlp.fc2.bias"] = r(width, mlp), torch.zeros(width)


class VisionTower:
    tower_id = "vision"

    def __init__(self, cfg: VisionTowerConfig, weights: dict[str, torch.Tensor], device: str | torch.device = "cpu",
                 dtype: torch.dtype | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.w = {k: v.to(self.device, self.dtype) for k, v in weights.items()}
        self.enc = _Encoder(self.w, cfg.depth, cfg.heads, cfg.eps)

    @staticmethod
    def random_weights(cfg: VisionTowerConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        w: dict[str, torch.Tensor] = {"patch_embed.weight": torch.randn(cfg.width, cfg.patch_dim, generator=g) * std,
                                      "patch_embed.bias": torch.zeros(cfg.width)}
        _init_blocks(w, cfg.depth, cfg.width, cfg.mlp, g, std)
        cell = cfg.width * cfg.merge * cfg.merge
        w["merger.norm.weight"], w["merger.norm.bias"] = torch.ones(cfg.width), torch.zeros(cfg.width)
        w["merger.fc1.weight"], w["merger.fc1.bias"] = torch.randn(cell, cell, generator=g) * std, torch.zeros(cell)
        w["merger.fc2.weight"], w["merger.fc2.bias"] = torch.randn(cfg.out_hidden, cell, generator=g) * std, torch.zeros(cfg.out_hidden)
        return w

    def rows_for(self, grid: tuple[int, int]) -> int:
        return grid[0] * grid[1] // (self.cfg.merge ** 2)

    @torch.no_grad()
    def forward(self, patches: torch.Tensor, grid: tuple[int, int]) -> torch.Tensor:
        """patches [gh * gw, 3 * p * p] (cell-major) -> [gh * gw / merge^2, out_hidden]."""
        cfg, w = self.cfg, self.w
        x = patches.to(self.device, self.dtype)
        x = _linear(x, w["patch_embed.weight"], w["patch_embed.bias"])
        pos = patch_positions(grid[0], grid[1], cfg.merge).to(self.device)
        rope = _rope_2d(pos, cfg.width // cfg.heads)
        for i in range(cfg.depth):
            x = self.enc.block(i, x, rope)
        x = F.layer_norm(x, (cfg.width,), w["merger.norm.weight"], w["merger.norm.bias"], cfg.eps)
        x = x.view(-1, cfg.width * cfg.merge * cfg.merge)                  # cell-major rows: one cell = consecutive patches
        x = F.gelu(_linear(x, w["merger.fc1.weight"], w["merger.fc1.bias"]))
        return _linear(x, w["merger.fc2.weight"], w["merger.fc2.bias"])


class AudioTower:
    tower_id = "audio"

    def __init__(self, cfg: AudioTowerConfig, weights: dict[str, torch.Tensor], device: str | torch.device = "cpu",
                 dtype: torch.dtype | None = None):
        self.cfg = cfg
        self.device = torch.device(device)
        self.dtype = dtype or (torch.bfloat16 if self.device.type == "cuda" else torch.float32)
        self.w = {k: v.to(self.device, self.dtype) for k, v in weights.items()}
        self.enc = _Encoder(self.w, cfg.depth, cfg.heads, cfg.eps)

    @staticmethod
    def random_weights(cfg: AudioTowerConfig, seed: int = 0, std: float = 0.02) -> dict[str, torch.Tensor]:
        g = torch.Generator().manual_seed(seed)
        w: dict[str, torch.Tensor] = {"conv1.weight": torch.randn(cfg.width, cfg.mels, 3, generator=g) * std,
                                      "conv1.bias": torch.zeros(cfg.width),
                                      "conv2.weight": torch.randn(cfg.width, cfg.width, 3, generator=g) * std,
                                      "conv2.bias": torch.zeros(cfg.width)}
        _init_blocks(w, cfg.depth, cfg.width, cfg.mlp, g, std)
        w["ln_post.weight"], w["ln_post.bias"] = torch.ones(cfg.width), torch.zeros(cfg.width)
        w["proj.weight"], w["proj.bias"] = torch.randn(cfg.out_hidden, cfg.width, generator=g) * std, torch.zeros(cfg.out_hidden)
        return w

    @staticmethod
    def rows_for_frames(frames: int) -> int:
        after_conv = (frames + 1) // 2            # conv2 has stride 2
        return max(1, after_conv // 2)            # average pooling by two

    @torch.no_grad()
    def forward(self, mel: torch.Tensor) -> torch.Tensor:
        """mel [frames, mels] -> [rows_for_frames(frames), out_hidden]."""
        cfg, w = self.cfg, self.w
        x = mel.to(self.device, self.dtype).T[None]                         # [1, mels, frames]
        x = F.gelu(F.conv1d(x, w["conv1.weight"], w["conv1.bias"], padding=1))
        x = F.gelu(F.conv1d(x, w["conv2.weight"], w["conv2.bias"], stride=2, padding=1))[0].T.contiguous()   # [n, width]
        n = x.shape[0]
        half = cfg.width // 2
        inv = torch.exp(-math.log(10000.0) * torch.arange(half, dtype=torch.float32, device=self.device) / max(1, half - 1))
        ang = torch.arange(n, dtype=torch.float32, device=self.device)[:, None] * inv[None]
        x = x + torch.cat([ang.sin(), ang.cos()], dim=1).to(self.dtype)
        for i in range(cfg.depth):
            x = self.enc.block(i, x, None)
        if n >= 2:
            x = x[: n // 2 * 2].view(n // 2, 2, cfg.width).mean(dim=1)
        x = F.layer_norm(x, (cfg.width,), w["ln_post.weight"], w["ln_post.bias"], cfg.eps)
        return _linear(x, w["proj.weight"], w["proj.bias"])
