"""Load the towers a checkpoint bundles.  Tensor names follow the Qwen-VL layout (``visual.patch_embed.proj``,
``visual.blocks.N.{norm1,norm2,attn.qkv,attn.proj,mlp.fc1,mlp.fc2}``, ``visual.merger.{ln_q,mlp.0,mlp.2}``) and the
Whisper-style audio layout (``audio_tower.{conv1,conv2,layers.N...,ln_post}``, ``audio_tower.proj``); a checkpoint
without them yields (None, None).  Geometry is read from the tensors' shapes."""
from __future__ import annotations

import torch

from ..loader.safetensors_io import Catalog
from .towers import AudioTower, AudioTowerConfig, VisionTower, VisionTowerConfig


def _vision(cat: Catalog, hidden: int, device) -> VisionTower | None:
    pre = next((p for p in ("visual.", "model.visual.", "vision_tower.") if f"{p}patch_embed.proj.weight" in cat), None)
    if pre is None:
        return None
    pe = cat.read(pre + "patch_embed.proj.weight").float()
    width = pe.shape[0]
    if pe.dim() == 5:                      # [width, 3, temporal, p, p]: a still image fills every temporal slot
        pe = pe.sum(dim=2)
    patch = pe.shape[-1]
    w: dict[str, torch.Tensor] = {"patch_embed.weight": pe.reshape(width, -1),
                                  "patch_embed.bias": cat.read(pre + "patch_embed.proj.bias").float()
                                  if pre + "patch_embed.proj.bias" in cat else torch.zeros(width)}
    depth = 0
    while f"{pre}blocks.{depth}.attn.qkv.weight" in cat:
        for name in ("norm1.weight", "norm1.bias", "norm2.weight", "norm2.bias", "attn.qkv.weight", "attn.qkv.bias",
                     "attn.proj.weight", "attn.proj.bias", "mlp.fc1.weight", "mlp.fc1.bias", "mlp.fc2.weight", "mlp.fc2.bias"):
            src = f"{pre}blocks.{depth}.{name}"
            if src in cat:
                w[f"blocks.{depth}.{name}"] = cat.read(src).float()
            else:                            # norms without a bias, projections without a bias
                ref = w[f"blocks.{depth}.{name.replace('bias', 'weight')}"]
                w[f"blocks.{depth}.{name}"] = torch.zeros(ref.shape[0])
        depth += 1
    mlp = w["blocks.0.mlp.fc1.weight"].shape[0]
    fc1 = cat.read(pre + "merger.mlp.0.weight").float()
    merge = int(round((fc1.shape[1] // width) ** 0.5))
    w["merger.norm.weight"] = cat.read(pre + "merger.ln_q.weight").float()
    w["merger.norm.bias"] = cat.read(pre + "merger.ln_q.bias").float() if pre + "merger.ln_q.bias" in cat else torch.zeros(width)
    w["merger.fc1.weight"], w["merger.fc1.bias"] = fc1, cat.read(pre + "merger.mlp.0.bias").float()
    w["merger.fc2.weight"], w["merger.fc2.bias"] = cat.read(pre + "merger.mlp.2.weight").float(), cat.read(pre + "merger.mlp.2.bias").float()
    out_hidden = w["merger.fc2.weight"].shape[0]
    if out_hidden != hidden:
        raise ValueError(f"vision tower projects to {out_hidden}, the language model is {hidden} wide")
    heads = max(1, width // 80) if width % 80 == 0 else max(1, width // 64)
    cfg = VisionTowerConfig(patch=patch, merge=merge, width=width, depth=depth, heads=heads, mlp=mlp, out_hidden=out_hidden)
    return VisionTower(cfg, w, device)


def _audio(cat: Catalog, hidden: int, device) -> AudioTower | None:
    pre = next((p for p in ("audio_tower.", "model.audio_tower.") if f"{p}conv1.weight" in cat), None)
    if pre is None or f"{pre}proj.weight" not in cat:
        return None
    w = {k[len(pre):]: cat.read(k).float() for k in cat.names() if k.startswith(pre)}
    width, mels = w["conv1.weight"].shape[0], w["conv1.weight"].shape[1]
    depth = 0
    while f"blocks.{depth}.attn.qkv.weight" in w:
        depth += 1
    if depth == 0:
        return None
    cfg = AudioTowerConfig(mels=mels, width=width, depth=depth, heads=max(1, width // 64), mlp=w["blocks.0.mlp.fc1.weight"].shape[0],
                           out_hidden=w["proj.weight"].shape[0])
    if cfg.out_hidden != hidden:
        raise ValueError(f"audio tower projects to {cfg.out_hidden}, the language model is {hidden} wide")
    return AudioTower(cfg, w, device)


def load_towers(snapshot_dir: str, hidden: int, device="cpu"):
    from ..loader.snapshot import resolve
    cat = Catalog(resolve(snapshot_dir))
    try:
        return _vision(cat, hidden, device), _audio(cat, hidden, device)
    finally:
        cat.close()
