"""Checkpoint quantisation pipeline: a bf16 (or any decodable) snapshot in, a snapshot in a serving format out.

    python -m cuteafd_b200.cli quantize <src> <dst> --experts exl3_k4 --attention fp8_block128

A recipe names one format per role (routed_expert, shared_expert, dense_ffn, attention, indexer, mtp); norms, the
router, the embedding and the head always stay as stored, because the engines serve them in bf16 / f32.  Every
operand is decoded with the loader's oracle decoder, re-encoded with the encoder of its target format and written
with the tensor names the format detector recognises, so the output needs no side file to be served.

Work is split by operand across ``world`` workers (one process per GPU of the box, or several CPU processes); worker
``rank`` encodes the operands ``rank, rank + world, ...`` of the sorted list and writes its own shard files, and the
last step merges the per-worker indexes into ``model.safetensors.index.json``.  Encoders run on ``device``: the EXL3
trellis search is plain tensor code and runs on a GPU as well as on the CPU.

A manifest (``quantization.json``) records the recipe, per-operand relative error and the sha256 of every source
tensor, which is what makes a re-run resumable (finished operands are skipped when their source hash matches).

Counterparts: quantization/*.py (distributed EXL3 quantisation and packaging), python/cuteafd_runtime/
exl3_quantizer.py, quantization/ple_nvfp4_cpu.cpp (CPU NVFP4 encoder) of the reference.
"""
from __future__ import annotations

import json
import os
import shutil
from dataclasses import dataclass, field

import torch

from ..loader import families, formats, snapshot
from ..loader.safetensors_io import Catalog, write_file
from . import codecs, exl3_encode

QUANT_ROLES = ("routed_expert", "shared_expert", "dense_ffn", "attention", "indexer", "mtp")
FORMATS = ("keep", "bf16", "fp8_block128", "nvfp4", "mxfp4", "exl3_k2", "exl3_k3", "exl3_k4", "exl3_k5", "exl3_k6", "exl3_k8")


@dataclass
class Recipe:
    """Target format per role; "keep" leaves the stored tensors untouched."""
    roles: dict[str, str] = field(default_factory=dict)
    seed: int = 0

    def __post_init__(self) -> None:
        for role, fmt in self.roles.items():
            if role not in QUANT_ROLES:
                raise ValueError(f"role {role!r} cannot be quantised (choose from {', '.join(QUANT_ROLES)})")
            if fmt not in FORMATS:
                raise ValueError(f"unknown format {fmt!r} (choose from {', '.join(FORMATS)})")

    def target(self, role: str) -> str:
        return self.roles.get(role, "keep")


def encode_operand(w: torch.Tensor, fmt: str, prefix: str, seed: int = 0, device: str | torch.device = "cpu",
                   hessian: torch.Tensor | None = None) -> tuple[dict[str, torch.Tensor], float]:
    """Encode an [out, in] fp32 weight; returns (tensors to store, relative error of the decoded result).  ``hessian``
    [in, in] (sum of x x^T over calibration inputs of this projection) is used by the EXL3 encoder's error feedback."""
    w = w.float()
    if fmt.startswith("exl3"):
        bits = int(fmt.split("k")[-1])
        r = exl3_encode.exl3_quantize(w.T.contiguous(), bits, torch.Generator().manual_seed(seed), device=device,
                                      hessian=hessian)
        return ({f"{prefix}.trellis": r["trellis"], f"{prefix}.suh": r["suh"], f"{prefix}.svh": r["svh"]},
                float(r["proxy_error"]))
    out = formats.encode(w, fmt, prefix)
    if fmt == "bf16":
        back = out[f"{prefix}.weight"].float()
    elif fmt == "fp8_block128":
        back = codecs.fp8_dequant_block128(out[f"{prefix}.weight"], out[f"{prefix}.weight_scale_inv"])
    elif fmt == "nvfp4":
        back = codecs.nvfp4_dequant(out[f"{prefix}.weight"], out[f"{prefix}.weight_scale"], out[f"{prefix}.weight_scale_2"])
    else:
        back = codecs.mxfp4_dequant(out[f"{prefix}.weight"], out[f"{prefix}.weight_scale"])
    err = ((back.float() - w).pow(2).sum() / w.pow(2).sum().clamp_min(1e-30)).sqrt()
    return out, float(err)


def _eligible(op: formats.QuantOperand, fmt: str) -> bool:
    n, k = op.shape
    if fmt.startswith("exl3"):
        return n % 128 == 0 and k % 128 == 0
    if fmt == "fp8_block128":
        return k % 128 == 0
    if fmt in ("nvfp4", "mxfp4"):
        return k % 32 == 0
    return True


def quantize_snapshot(src: str, dst: str, recipe: Recipe, rank: int = 0, world: int = 1,
                      device: str | torch.device = "cpu", log=print, hessians: str | None = None) -> dict:
    """Run worker ``rank`` of ``world``.  Returns this worker's manifest part; rank 0 also merges (see ``merge``).
    ``hessians``: a directory of safetensors files holding ``<operand prefix>.hessian`` [in, in] tensors from a
    calibration run; operands that have one are encoded with error feedback (EXL3 targets)."""
    hcat = Catalog(hessians) if hessians else None
    src = snapshot.resolve(src)
    cfg, hf = snapshot.read_config(src)
    fam = families.detect(hf)
    if fam is None:
        raise ValueError("no family recognises this checkpoint")
    model = fam.open(cfg, hf)
    cat = Catalog(src)
    ops = formats.detect_operands(cat)
    os.makedirs(dst, exist_ok=True)
    part_path = os.path.join(dst, f"quantization.part{rank}.json")
    done: dict = {}
    if os.path.exists(part_path):
        with open(part_path) as f:
            done = json.load(f).get("operands", {})
    owned = set()
    for op in ops.values():
        owned.update(n for n in (op.weight, op.scale_tensor, op.global_scale, op.input_scale, *op.companions.values()) if n)
    todo = []
    for pre in sorted(ops):
        role = model.classify(ops[pre].weight)[0]
        fmt = recipe.target(role) if role in QUANT_ROLES else "keep"
        if fmt != "keep" and not _eligible(ops[pre], fmt):
            fmt = "keep"
        todo.append((pre, role, fmt))
    mine = todo[rank::world]
    tensors: dict[str, torch.Tensor] = {}
    report: dict = {}
    for pre, role, fmt in mine:
        op = ops[pre]
        names = [n for n in (op.weight, op.scale_tensor, op.global_scale, op.input_scale, *op.companions.values()) if n]
        if fmt == "keep" or fmt == op.format:
            for n in names:
                tensors[n] = cat.read(n)
            report[pre] = {"role": role, "format": op.format, "kept": True}
            continue
        digest = cat.sha256(op.weight)
        prev = done.get(pre)
        shard_prev = os.path.join(dst, prev["file"]) if prev and "file" in prev else None
        if prev and prev.get("source_sha256") == digest and prev.get("format") == fmt and shard_prev and os.path.exists(shard_prev):
            report[pre] = prev
            continue
        w = formats.dequantize(op, cat)
        hess = hcat.read(pre + ".hessian").double() if hcat is not None and (pre + ".hessian") in hcat else None
        enc, err = encode_operand(w, fmt, pre, seed=recipe.seed + len(report), device=device, hessian=hess)
        fname = f"quant-{rank:03d}-{len(report):06d}.safetensors"
        write_file(os.path.join(dst, fname), enc, {"format": "pt"})
        report[pre] = {"role": role, "format": fmt, "rel_error": err, "source_sha256": digest, "file": fname,
                       "tensors": sorted(enc), "calibrated": hess is not None}
        log(f"[quantize r{rank}] {pre}: {op.format} -> {fmt}  rel err {err:.4f}")
        with open(part_path, "w") as f:
            json.dump({"operands": report}, f)
    # tensors that belong to no operand (biases, 1-D parameters) go with rank 0
    if rank == 0:
        for n in cat.names():
            if n not in owned:
                tensors[n] = cat.read(n)
    if tensors:
        fname = f"kept-{rank:03d}.safetensors"
        write_file(os.path.join(dst, fname), tensors, {"format": "pt"})
        report["__kept__"] = {"file": fname, "tensors": sorted(tensors)}
    with open(part_path, "w") as f:
        json.dump({"operands": report}, f)
    cat.close()
    return report


def merge(src: str, dst: str, recipe: Recipe, world: int = 1) -> dict:
    """Write the weight index, the manifest and the side files once every worker has finished."""
    src = snapshot.resolve(src)
    weight_map: dict[str, str] = {}
    operands: dict = {}
    for r in range(world):
        with open(os.path.join(dst, f"quantization.part{r}.json")) as f:
            part = json.load(f)["operands"]
        for pre, rec in part.items():
            for n in rec.get("tensors", []):
                weight_map[n] = rec["file"]
            if pre != "__kept__":
                operands[pre] = {k: v for k, v in rec.items() if k != "tensors"}
    total = sum(os.path.getsize(os.path.join(dst, f)) for f in set(weight_map.values()))
    with open(os.path.join(dst, "model.safetensors.index.json"), "w") as f:
        json.dump({"metadata": {"total_size": total}, "weight_map": weight_map}, f, indent=1, sort_keys=True)
    for side in os.listdir(src):
        if side.endswith(".safetensors") or side == "model.safetensors.index.json":
            continue
        p = os.path.join(src, side)
        if os.path.isfile(p):
            shutil.copy(p, os.path.join(dst, side))
    errs = [v["rel_error"] for v in operands.values() if "rel_error" in v]
    manifest = {"recipe": recipe.roles, "seed": recipe.seed, "operands": operands,
                "summary": {"quantised": len(errs), "kept": len(operands) - len(errs),
                            "max_rel_error": max(errs) if errs else 0.0,
                            "mean_rel_error": sum(errs) / len(errs) if errs else 0.0, "bytes": total}}
    with open(os.path.join(dst, "quantization.json"), "w") as f:
        json.dump(manifest, f, indent=1, sort_keys=True)
    return manifest


def run(src: str, dst: str, recipe: Recipe, device: str | torch.device = "cpu", log=print) -> dict:
    """Single-process convenience: one worker, then the merge."""
    quantize_snapshot(src, dst, recipe, 0, 1, device, log)
    return merge(src, dst, recipe, 1)
