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
                only: str | None = None) -> tuple[ModelConfig, dict[str, torch.Tensor]]:
    """Every parameter decoded to a dense tensor under its ``....weight`` name."""
    snap = open_snapshot(path)
    out: dict[str, torch.Tensor] = {}
    covered = set()
    for pre, op in snap.operands.items():
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
                            expert_range: tuple[int, int] | None = None):
    """Device weights for ``GqaMoeEngine`` straight from a snapshot (bf16 compute form)."""
    from ..models.gqa_moe import GqaMoeWeights, LayerWeights
    snap = open_snapshot(path)
    cfg, cat, ops = snap.cfg, snap.catalog, snap.operands

    def dense(prefix: str) -> torch.Tensor:
        return formats.dequantize(ops[prefix], cat).to(torch.bfloat16).to(device).contiguous()

    def raw(name: str, dt=torch.bfloat16) -> torch.Tensor:
        return cat.read(name).to(dt).to(device).contiguous()

    W = GqaMoeWeights(cfg)
    W.embed, W.final_norm = raw("model.embed_tokens.weight"), raw("model.norm.weight")
    W.lm_head = W.embed if cfg.tie_embeddings else raw("lm_head.weight")
    lo, hi = expert_range or (0, cfg.num_experts)
    for i in range(cfg.num_layers):
        pre, L = f"model.layers.{i}.", LayerWeights()
        a, m = pre + "self_attn.", pre + "mlp."
        L.ln1, L.ln2 = raw(pre + "input_layernorm.weight"), raw(pre + "post_attention_layernorm.weight")
        L.wqkv = torch.cat([dense(a + "q_proj"), dense(a + "k_proj"), dense(a + "v_proj")]).contiguous()
        L.wo = dense(a + "o_proj")
        if cfg.qk_norm:
            L.q_norm, L.k_norm = raw(a + "q_norm.weight"), raw(a + "k_norm.weight")
        if cfg.is_moe_layer(i):
            L.router = raw(m + "gate.weight")
            bn = m + "gate.e_score_correction_bias"
            L.router_bias = raw(bn, torch.float32) if bn in cat else None
            if with_experts:
                for dst, src in (("w_gate", "gate_proj"), ("w_up", "up_proj"), ("w_down", "down_proj")):
                    setattr(L, dst, torch.stack([dense(f"{m}experts.{e}.{src}") for e in range(lo, hi)]).contiguous())
            if cfg.num_shared_experts:
                L.s_gate, L.s_up, L.s_down = (dense(f"{m}shared_experts.{n}_proj") for n in ("gate", "up", "down"))
        else:
            L.d_gate, L.d_up, L.d_down = (dense(f"{m}{n}_proj") for n in ("gate", "up", "down"))
        W.layers.append(L)
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
