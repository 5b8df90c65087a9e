"""Family registry: static descriptors that detect a checkpoint's family, open it into a typed
model description, classify every tensor into a component role, and say which stored formats the
engine has kernels for.  An unsupported operand is a *result* (a ``Hint`` saying what is missing
and what would fix it), never an exception.

Counterpart: rust/crates/cuteafd-loader/src/plan/family.rs:19-256 (Hint, ExpertContract,
FamilyModel, Family, REGISTRY, detect) and plan/spec.rs (Component roles).
"""
from __future__ import annotations

import re
from dataclasses import dataclass, field

from ..config import ModelConfig
from .formats import QuantOperand

ROLES = ("embedding", "head", "final_norm", "norm", "attention", "indexer", "router", "routed_expert",
         "shared_expert", "dense_ffn", "mtp", "other")


@dataclass(frozen=True)
class Hint:
    what: str      # what cannot be served as stored
    how: str       # what would make it servable


@dataclass
class ExpertContract:
    """What the expert ranks of this family must provide."""
    activation: str = "silu"
    formats: tuple[str, ...] = ("bf16", "fp8_block128", "nvfp4", "mxfp4", "exl3")
    wire: str = "bf16"
    slice_granule: int = 128


@dataclass
class FamilyModel:
    family: "Family"
    cfg: ModelConfig
    contract: ExpertContract = field(default_factory=ExpertContract)

    _LAYER = re.compile(r"model\.layers\.(\d+)\.(.*)")

    def classify(self, name: str) -> tuple[str, int | None, int | None]:
        """(role, layer, expert) of a tensor name."""
        if name.startswith("model.embed_tokens"):
            return "embedding", None, None
        if name.startswith("lm_head"):
            return "head", None, None
        if name.startswith("model.norm"):
            return "final_norm", None, None
        m = self._LAYER.match(name)
        if not m:
            return "other", None, None
        layer, rest = int(m.group(1)), m.group(2)
        if layer >= self.cfg.num_layers and not rest.startswith("mlp.experts"):
            return "mtp", layer, None
        if "indexer" in rest:
            return "indexer", layer, None
        if rest.startswith("self_attn"):
            return "attention", layer, None
        if rest.startswith("mlp.experts."):
            return "routed_expert", layer, int(rest.split(".")[2])
        if rest.startswith("mlp.shared_expert"):
            return "shared_expert", layer, None
        if rest.startswith("mlp.gate.") :
            return "router", layer, None
        if rest.startswith("mlp."):
            return "dense_ffn", layer, None
        if "norm" in rest:
            return "norm", layer, None
        return "other", layer, None

    def accepts(self, op: QuantOperand, role: str) -> Hint | None:
        """None when the engine serves this operand as stored; otherwise the reason."""
        fmt = op.format.split("_k")[0] if op.format.startswith("exl3") else op.format
        if role in ("embedding", "head", "final_norm", "norm", "router"):
            if op.encoding not in ("bf16", "f16", "f32"):
                return Hint(f"{op.name}: {role} stored as {op.format}", "store norms, router, embedding and head in bf16/f32")
            return None
        if role == "routed_expert":
            if fmt not in self.contract.formats:
                return Hint(f"{op.name}: routed expert stored as {op.format}",
                            f"supported expert formats: {', '.join(self.contract.formats)}")
            if op.shape[1] % 128 and fmt != "bf16":
                return Hint(f"{op.name}: K={op.shape[1]} is not a multiple of 128", "pad the expert intermediate to whole 128 blocks")
            return None
        if fmt not in ("bf16", "f16", "f32", "fp8_block128", "nvfp4", "mxfp4", "exl3"):
            return Hint(f"{op.name}: {role} stored as {op.format}", "no decoder for this encoding")
        return None


class Family:
    """Static descriptor.  Subclasses set ``id`` and ``model_types`` and may refine ``open``."""
    id = ""
    model_types: tuple[str, ...] = ()
    attention = "mla"
    speculators: tuple[str, ...] = ("off",)
    decode_lanes = (1, 2)
    prefill_unit_rows = 2752
    max_context = 1 << 20

    def detect(self, hf_config: dict) -> bool:
        return hf_config.get("model_type") in self.model_types

    def open(self, cfg: ModelConfig, hf_config: dict) -> FamilyModel:
        return FamilyModel(self, cfg)


class DeepseekV3(Family):
    id, model_types = "deepseek_v3", ("deepseek_v3", "deepseek_v2", "kimi_k2")
    speculators = ("off", "mtp")

    def detect(self, hf_config: dict) -> bool:
        return super().detect(hf_config) and not hf_config.get("index_n_heads")


class DeepseekV32(Family):
    id, model_types = "deepseek_v32", ("deepseek_v32", "deepseek_v3", "glm_moe_dsa")
    speculators = ("off", "mtp")

    def detect(self, hf_config: dict) -> bool:
        return hf_config.get("model_type") in self.model_types and bool(hf_config.get("index_n_heads"))


class Qwen3Moe(Family):
    id, model_types, attention = "qwen3_moe", ("qwen3_moe", "qwen2_moe", "mixtral", "qwen3"), "gqa"


class Llama(Family):
    """Dense GQA decoders (Llama; Mistral, sliding-window layers included): served by the GQA engine's dense path."""
    id, model_types, attention = "llama", ("llama", "mistral"), "gqa"


class Glm4Moe(Family):
    """GLM-4.5 / 4.6 (glm4_moe): GQA with biased q / k / v and partial rotary, sigmoid routing with a correction bias, a
    shared expert and an MTP depth; served by the GQA engine."""
    id, model_types, attention = "glm4_moe", ("glm4_moe",), "gqa"
    speculators = ("off", "mtp")


class Qwen2(Family):
    """Dense Qwen2 / Qwen2.5 decoders (biased q / k / v): the GQA engine's dense path."""
    id, model_types, attention = "qwen2", ("qwen2",), "gqa"


class TinyMoe(Family):
    id, model_types = "tiny_moe", ("tiny_moe",)


_ALIASES = ((".block_sparse_moe.gate.", ".mlp.gate."), (".block_sparse_moe.experts.", ".mlp.experts."),
            (".mlp.shared_expert.", ".mlp.shared_experts."))
_MIXTRAL_PROJ = {"w1": "gate_proj", "w3": "up_proj", "w2": "down_proj"}
_MIXTRAL_RE = re.compile(r"(\.mlp\.experts\.\d+\.)(w[123])(\.)")


def canonical_name(name: str) -> str:
    """Checkpoint tensor name -> the name the loaders use.  Mixtral-style files call the MoE block
    ``block_sparse_moe`` and its projections ``w1 / w3 / w2`` (gate / up / down); Qwen2-MoE says ``shared_expert``."""
    for a, b in _ALIASES:
        if a in name:
            name = name.replace(a, b)
    return _MIXTRAL_RE.sub(lambda m: m.group(1) + _MIXTRAL_PROJ[m.group(2)] + m.group(3), name)


REGISTRY: tuple[Family, ...] = (DeepseekV32(), DeepseekV3(), Qwen3Moe(), Glm4Moe(), Qwen2(), Llama(), TinyMoe())


def detect(hf_config: dict) -> Family | None:
    for fam in REGISTRY:
        if fam.detect(hf_config):
            return fam
    return None


def by_id(fid: str) -> Family:
    for fam in REGISTRY:
        if fam.id == fid:
            return fam
    raise KeyError(fid)
