"""Open a snapshot: config + catalog + operands + family, and materialise weights.

``open_snapshot`` is header-only (planning).  ``load_params`` decodes every operand to a dense
tensor keyed by Hugging Face names (oracle and bf16 engine path).  ``load_gqa_engine_weights``
builds the device-resident weight set of the GQA MoE engine, streaming one layer at a time so
host memory holds one layer, not the model (the reference streams shards to its ranks the same
way: rust/crates/cuteafd-loader/src/push_load.rs).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config import ModelConfig
from . import families, formats
from .safetensors_io import Catalog
from .snapshot import read_config, resolve


@dataclass
class OpenedSnapshot:
    path: str
    cfg: ModelConfig
    hf_config: dict
    catalog: Catalog
    operands: dict[str, formats.QuantOperand]
    family: families.Family | None
    model: families.FamilyModel | None

    def hints(self) -> list[families.Hint]:
        if self.model is None:
            return [families.Hint(f"model_type {self.hf_config.get('model_type')!r} matches no family",
                                  "supported families: " + ", ".join(f.id for f in families.REGISTRY))]
        out = []
        for op in self.operands.values():
            role, _, _ = self.model.classify(op.weight)
            h = self.model.accepts(op, role)
            if h:
                out.append(h)
        return out


def open_snapshot(path: str) -> OpenedSnapshot:
    path = resolve(path)
    cfg, hf = read_config(path)
    cat = Catalog(path, rename=families.canonical_name)
    ops = formats.detect_operands(cat)
    fam = families.detect(hf)
    model = fam.open(cfg, hf) if fam else None
    return OpenedSnapshot(path, cfg, hf, cat, ops, fam, model)


def load_params(path: str, dtype: torch.dtype = torch.float32, device: str = "cpu",
                only: str | None = None, exclude: str | None = None, keep=None) -> tuple[ModelConfig, dict[str, torch.Tensor]]:
    """Every parameter decoded to a dense tensor under its ``....weight`` name.  ``only`` / ``exclude`` keep or drop
    the operands whose prefix contains the substring (an expert rank reads ``only=".mlp.experts."``, the attention rank
    of a disaggregated deployment ``exclude=".mlp.experts."``); ``keep(prefix) -> bool`` is the general form (an expert
    rank that reads only its own expert range).  Dropped operands are not read at all."""
    snap = open_snapshot(path)
    out: dict[str, torch.Tensor] = {}
    covered = set()
    for pre, op in snap.operands.items():
        if (exclude and exclude in pre) or (keep is not None and not keep(pre)):
            covered.update(n for n in (op.weight, op.scale_tensor, op.global_scale, op.input_scale, *op.companions.values()) if n)
            continue
        if only and only not in pre:
            continue
        names = [op.weight, op.scale_tensor, op.global_scale, op.input_scale, *op.companions.values()]
        covered.update(n for n in names if n)
        out[pre + ".weight"] = formats.dequantize(op, snap.catalog, device).to(dtype)
    for name in snap.catalog.names():
        if name not in covered and (not only or only in name):
            t = snap.catalog.read(name)
            out[name] = t.to(device=device, dtype=dtype if t.is_floating_point() and "bias" not in name else t.dtype)
    return snap.cfg, out


def load_gqa_engine_weights(path: str, device: torch.device, with_experts: bool = True,
                            expert_range: tuple[int, int] | None = None, reserve_bytes: int = 0):
    """Device weights for ``GqaMoeEngine`` straight from a snapshot (bf16 compute form), in one weight arena.

    Two passes over the same item list: the first only reads shapes from the catalog and reserves a slot per engine
    tensor (fused q/k/v rows, stacked experts), the arena is checked against the device's free memory (less
    ``reserve_bytes`` for KV and workspaces) and allocated once, and the second decodes every stored tensor and copies
    it straight into its rows of its slot, so no concatenated or stacked temporary ever exists on the device."""
    from ..models.gqa_moe import GqaMoeWeights, LayerWeights
    from ..runtime.arena import WeightArena
    snap = open_snapshot(path)
    cfg, cat, ops = snap.cfg, snap.catalog, snap.operands
    device = torch.device(device)
    arena = WeightArena(device, owner=f"gqa:{cfg.name}")
    items: list = []
    bf16 = torch.bfloat16

    def shape_of(part) -> tuple[int, ...]:
        kind, name = part
        return tuple(ops[name].shape) if kind == "dense" else tuple(cat.entries[name].shape)

    def want(obj, attr: str, slot: str, parts: list, mode: str = "cat", dt: torch.dtype = bf16) -> None:
        shapes = [shape_of(p) for p in parts]
        shape = (len(parts), *shapes[0]) if mode == "stack" else (sum(s[0] for s in shapes), *shapes[0][1:])
        arena.reserve(slot, shape, dt)
        items.append((obj, attr, slot, parts, mode, dt))

    W = GqaMoeWeights(cfg)
    want(W, "embed", "embed", [("raw", "model.embed_tokens.weight")])
    want(W, "final_norm", "final_norm", [("raw", "model.norm.weight")])
    if not cfg.tie_embeddings:
        want(W, "lm_head", "lm_head", [("raw", "lm_head.weight")])
    lo, hi = expert_range or (0, cfg.num_experts)
    for i in range(cfg.num_layers):
        pre, L = f"model.layers.{i}.", LayerWeights()
        a, m, s = pre + "self_attn.", pre + "mlp.", f"layers.{i}."
        want(L, "ln1", s + "ln1", [("raw", pre + "input_layernorm.weight")])
        want(L, "ln2", s + "ln2", [("raw", pre + "post_attention_layernorm.weight")])
        want(L, "wqkv", s + "wqkv", [("dense", a + "q_proj"), ("dense", a + "k_proj"), ("dense", a + "v_proj")])
        want(L, "wo", s + "wo", [("dense", a + "o_proj")])
        if cfg.qk_norm:
            want(L, "q_norm", s + "q_norm", [("raw", a + "q_norm.weight")])
            want(L, "k_norm", s + "k_norm", [("raw", a + "k_norm.weight")])
        if cfg.is_moe_layer(i):
            want(L, "router", s + "router", [("raw", m + "gate.weight")])
            bn = m + "gate.e_score_correction_bias"
            L.router_bias = None
            if bn in cat:
                want(L, "router_bias", s + "router_bias", [("raw", bn)], dt=torch.float32)
            if with_experts:
                for dst, src in (("w_gate", "gate_proj"), ("w_up", "up_proj"), ("w_down", "down_proj")):
                    want(L, dst, s + dst, [("dense", f"{m}experts.{e}.{src}") for e in range(lo, hi)], mode="stack")
            if cfg.num_shared_experts:
                for n in ("gate", "up", "down"):
                    want(L, "s_" + n, s + "s_" + n, [("dense", f"{m}shared_experts.{n}_proj")])
        else:
            for n in ("gate", "up", "down"):
                want(L, "d_" + n, s + "d_" + n, [("dense", f"{m}{n}_proj")])
        W.layers.append(L)

    if device.type == "cuda":
        arena.check_fits(torch.cuda.mem_get_info(device)[0], reserve_bytes)
    arena.allocate()
    for obj, attr, slot, parts, mode, dt in items:
        row = 0
        for kind, name in parts:
            t = formats.dequantize(ops[name], cat) if kind == "dense" else cat.read(name)
            t = t.to(dt)
            if mode == "stack":
                arena.fill_rows(slot, row, t[None].to(device))
                row += 1
            else:
                arena.fill_rows(slot, row, t.to(device))
                row += t.shape[0]
        setattr(obj, attr, arena.view(slot))
    left = arena.missing()
    if left:
        raise RuntimeError(f"weights left unwritten: {left[:4]}")
    if cfg.tie_embeddings:
        W.lm_head = W.embed
    W.arena = arena
    return cfg, W


def load_engine(path: str, device: torch.device, num_pages: int, max_tokens: int, max_seqs: int, kv_format: str = "auto"):
    """(cfg, engine) for a snapshot: the GQA engine streams its weights tensor by tensor; MLA checkpoints (and any
    checkpoint with MTP depths) go through the dense parameter dictionary, decoded to bf16.  ``kv_format`` "auto"
    picks the 656-byte FP8 latent record for sparse-attention (indexer) checkpoints and bf16 records otherwise."""
    snap = open_snapshot(path)
    cfg = snap.cfg
    if cfg.is_mla:
        want = ("fp8_ds_mla" if cfg.indexer_heads else "bf16") if kv_format == "auto" else kv_format
        if want == "fp8_ds_mla" and not cfg.indexer_heads:
            raise ValueError("fp8_ds_mla records need the sparse attention path (a checkpoint with an indexer)")
        cfg = cfg.replace(kv_format=want)
    if cfg.is_mla:
        from ..models.mla_moe import LatentCache, MlaMoeEngine, MlaMoeWeights
        _, params = load_params(path, dtype=torch.bfloat16)
        W = MlaMoeWeights.from_params(cfg, params, device)
        return cfg, MlaMoeEngine(cfg, W, LatentCache(cfg, num_pages, device), max_tokens=max_tokens, max_seqs=max_seqs)
    from ..models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
    if cfg.mtp_layers:
        _, params = load_params(path, dtype=torch.bfloat16)
        W = GqaMoeWeights.from_params(cfg, params, device)
    else:
        _, W = load_gqa_engine_weights(path, device)
    return cfg, GqaMoeEngine(cfg, W, KvCache(cfg, num_pages, device), max_tokens=max_tokens, max_seqs=max_seqs)
