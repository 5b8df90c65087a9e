"""Lossless description of how each weight is stored, detected from tensor names and dtypes.

A ``QuantOperand`` groups a weight with its companions (block scales, global scale, input scale,
trellis rotations) and names its encoding; nothing is repacked.  Counterpart:
rust/crates/cuteafd-loader/src/plan/format.rs:29-135 (Encoding, ScaleEncoding, RowTiling,
BlockScale, QuantOperand) and formats/{modelopt,exl3_storage,fp8_experts}.rs.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import torch

from ..quant import codecs
from .safetensors_io import Catalog, TensorEntry

ENCODINGS = ("bf16", "f16", "f32", "e4m3", "e5m2", "e2m1", "exl3", "int8")


@dataclass(frozen=True)
class BlockScale:
    encoding: str            # "f32" | "bf16" | "e4m3" | "ue8m0"
    rows: int                # weight rows covered by one scale (1 = per row)
    cols: int                # weight columns (K) covered by one scale
    direction: str = "multiply"   # stored value multiplies the decoded weight


@dataclass
class QuantOperand:
    name: str                              # tensor prefix, e.g. "model.layers.3.mlp.experts.7.down_proj"
    encoding: str
    shape: tuple[int, int]                 # logical [out_features, in_features]
    weight: str                            # tensor holding the payload
    block_scale: BlockScale | None = None
    scale_tensor: str | None = None
    global_scale: str | None = None        # fp32 scalar multiplier (NVFP4 weight_scale_2)
    input_scale: str | None = None
    bits: float = 16.0                     # payload bits per weight
    companions: dict[str, str] = field(default_factory=dict)

    @property
    def format(self) -> str:
        if self.encoding == "e4m3":
            return "fp8_block128"
        if self.encoding == "e2m1":
            return "nvfp4" if self.block_scale and self.block_scale.encoding == "e4m3" else "mxfp4"
        if self.encoding == "exl3":
            return f"exl3_k{self.bits:g}"
        return self.encoding

    def stored_bytes(self, cat: Catalog) -> int:
        names = [self.weight, self.scale_tensor, self.global_scale, self.input_scale, *self.companions.values()]
        return sum(cat.entries[n].nbytes for n in names if n and n in cat.entries)


def detect_operands(cat: Catalog) -> dict[str, QuantOperand]:
    """Group the catalog's tensors into operands keyed by prefix."""
    ops: dict[str, QuantOperand] = {}
    E = cat.entries
    for name, e in E.items():
        if name.endswith(".trellis"):
            pre = name[: -len(".trellis")]
            kt, nt, w = e.shape
            bits = w / 16
            comp = {k: f"{pre}.{k}" for k in ("suh", "svh", "mcg", "mul1") if f"{pre}.{k}" in E}
            ops[pre] = QuantOperand(pre, "exl3", (nt * 16, kt * 16), name, bits=bits, companions=comp)
        elif name.endswith(".weight"):
            pre = name[: -len(".weight")]
            if len(e.shape) != 2:
                ops[pre] = QuantOperand(pre, _plain(e), tuple(e.shape) if len(e.shape) == 2 else (e.shape[0], 1), name,
                                        bits=8.0 * e.nbytes / max(e.numel, 1))
                continue
            N, Kd = e.shape
            if e.dtype in ("F8_E4M3", "F8_E5M2"):
                sc = next((f"{pre}.{s}" for s in ("weight_scale_inv", "weight_scale") if f"{pre}.{s}" in E), None)
                bs = None
                if sc:
                    sr, scol = E[sc].shape if len(E[sc].shape) == 2 else (1, 1)
                    bs = BlockScale(_plain(E[sc]), max(1, -(-N // sr)) if sr else N, max(1, -(-Kd // scol)) if scol else Kd)
                    bs = BlockScale(bs.encoding, 128 if bs.rows > 1 else 1, 128 if bs.cols > 1 else Kd)
                ops[pre] = QuantOperand(pre, "e4m3" if e.dtype == "F8_E4M3" else "e5m2", (N, Kd), name, bs, sc, bits=8.0,
                                        input_scale=f"{pre}.input_scale" if f"{pre}.input_scale" in E else None)
            elif e.dtype == "U8" and f"{pre}.weight_scale" in E:
                sc = f"{pre}.weight_scale"
                se = E[sc]
                K_log = Kd * 2
                if se.dtype == "F8_E4M3":
                    bs = BlockScale("e4m3", 1, K_log // se.shape[1])
                else:
                    bs = BlockScale("ue8m0", 1, K_log // se.shape[1])
                ops[pre] = QuantOperand(pre, "e2m1", (N, K_log), name, bs, sc, bits=4.0,
                                        global_scale=f"{pre}.weight_scale_2" if f"{pre}.weight_scale_2" in E else None,
                                        input_scale=f"{pre}.input_scale" if f"{pre}.input_scale" in E else None)
            else:
                ops[pre] = QuantOperand(pre, _plain(e), (N, Kd), name, bits=8.0 * e.nbytes / max(e.numel, 1))
    return ops


def _plain(e: TensorEntry) -> str:
    return {"BF16": "bf16", "F16": "f16", "F32": "f32", "F8_E4M3": "e4m3", "F8_E5M2": "e5m2", "U8": "int8",
            "I8": "int8"}.get(e.dtype, e.dtype.lower())


def dequantize(op: QuantOperand, cat: Catalog, device: str | torch.device = "cpu") -> torch.Tensor:
    """Decode an operand to fp32 [out, in] (oracle path; the engine keeps the stored form)."""
    w = cat.read(op.weight).to(device)
    if op.encoding in ("bf16", "f16", "f32"):
        return w.float()
    if op.encoding in ("e4m3", "e5m2"):
        if op.scale_tensor is None:
            return w.float()
        s = cat.read(op.scale_tensor).to(device).float()
        if s.numel() == 1:
            return w.float() * s.reshape(())
        return codecs.fp8_dequant_block128(w, s)
    if op.encoding == "e2m1":
        s = cat.read(op.scale_tensor).to(device)
        if op.block_scale.encoding == "e4m3":
            g = cat.read(op.global_scale).to(device) if op.global_scale else torch.ones(1, device=device)
            return codecs.nvfp4_dequant(w, s, g, op.block_scale.cols)
        return codecs.mxfp4_dequant(w, s, op.block_scale.cols)
    if op.encoding == "exl3":
        suh = cat.read(op.companions["suh"]).to(device)
        svh = cat.read(op.companions["svh"]).to(device)
        return codecs.exl3_dequant(w, suh, svh).T.float()       # stored [in, out] -> [out, in]
    raise ValueError(f"{op.name}: no decoder for {op.encoding}")


def encode(w: torch.Tensor, fmt: str, prefix: str, gen: torch.Generator | None = None) -> dict[str, torch.Tensor]:
    """Encode an [out, in] weight into the tensors a snapshot of format ``fmt`` carries."""
    if fmt == "bf16":
        return {f"{prefix}.weight": w.to(torch.bfloat16)}
    if fmt == "fp8_block128":
        q, s = codecs.fp8_quant_block128(w)
        return {f"{prefix}.weight": q, f"{prefix}.weight_scale_inv": s}
    if fmt == "nvfp4":
        p, bs, g = codecs.nvfp4_quant(w)
        return {f"{prefix}.weight": p, f"{prefix}.weight_scale": bs, f"{prefix}.weight_scale_2": g,
                f"{prefix}.input_scale": torch.ones(1)}
    if fmt == "mxfp4":
        p, e = codecs.mxfp4_quant(w)
        return {f"{prefix}.weight": p, f"{prefix}.weight_scale": e}
    if fmt.startswith("exl3"):
        bits = int(fmt.split("k")[-1]) if "k" in fmt else 4
        t, suh, svh = codecs.exl3_random(w.shape[1], w.shape[0], bits, gen or torch.Generator().manual_seed(0))
        return {f"{prefix}.trellis": t, f"{prefix}.suh": suh, f"{prefix}.svh": svh}
    raise ValueError(f"unknown format {fmt}")
