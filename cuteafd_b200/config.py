"""Model geometry shared by the CPU oracle, the planner, the loader and the CUDA engine.

One dataclass describes every decoder family the engine serves: GQA or MLA attention,
dense or routed-MoE feed-forward layers, optional shared expert, optional multi-token
prediction (MTP) layers and the optional sparse-attention "lightning indexer".  The
reference keeps the same facts in ``ModelSpec/LayerSpec/AttentionKind/MoeSpec/
SpeculatorSpec`` (rust/crates/cuteafd-loader/src/plan/spec.rs:7-190).
"""
from __future__ import annotations

import dataclasses
import json
from dataclasses import dataclass, field
from typing import Any


@dataclass(frozen=True)
class ModelConfig:
    name: str = "tiny-moe"
    family: str = "deepseek_v3"          # deepseek_v3 | deepseek_v32 | qwen3_moe | glm4_moe | qwen2 | llama | tiny_moe
    vocab_size: int = 1024
    num_layers: int = 2
    hidden: int = 256
    # attention
    attention: str = "mla"               # "mla" | "gqa"
    num_heads: int = 4
    num_kv_heads: int = 4                # gqa only
    head_dim: int = 64                   # gqa only
    qk_norm: bool = False                # Qwen3: RMSNorm over head_dim on q and k
    rotary_dim: int = 0                  # gqa: leading dims of a head that are rotated (0 = all; GLM-4.5: half the head)
    attention_bias: bool = False         # gqa: q / k / v projections carry a bias (GLM-4.5, Qwen2)
    sliding_window: int = 0              # gqa: a query at position t sees keys (t - window, t] on the windowed layers (0 = none)
    window_layers: tuple = ()            # per layer, 1 = windowed; empty = every layer when sliding_window is set
    q_lora_rank: int = 128               # mla (0 = direct q projection)
    kv_lora_rank: int = 64
    qk_nope_dim: int = 32
    qk_rope_dim: int = 32
    v_head_dim: int = 32
    rope_theta: float = 10000.0
    rope_interleaved: bool = True        # pairs (2i, 2i+1); False = rotate-half (neox)
    # long-context frequency scaling of the checkpoint (config.json "rope_scaling"); see ref/ops.py::rope_inv_freq
    rope_scaling: str = "none"           # none | linear | llama3 | yarn
    rope_factor: float = 1.0
    rope_original_max: int = 4096        # positions the base frequencies were trained for (yarn, llama3)
    rope_beta_fast: float = 32.0         # yarn correction range
    rope_beta_slow: float = 1.0
    rope_mscale: float = 1.0             # yarn magnitude terms (DeepSeek: softmax scale *= mscale(all_dim)^2)
    rope_mscale_all_dim: float = 0.0
    rope_low_freq_factor: float = 1.0    # llama3
    rope_high_freq_factor: float = 4.0
    rms_eps: float = 1e-6
    # feed forward
    dense_ffn: int = 512                 # intermediate size of the dense SwiGLU layers
    first_dense_layers: int = 1          # layers [0, first_dense_layers) are dense
    num_experts: int = 8
    expert_ffn: int = 128
    top_k: int = 2
    scoring: str = "softmax"             # "softmax" | "sigmoid"
    num_groups: int = 1                  # group-limited routing (DeepSeek-V3: 8)
    topk_groups: int = 1                 # groups kept (DeepSeek-V3: 4)
    num_shared_experts: int = 1
    routed_scale: float = 1.0
    norm_topk_prob: bool = True
    router_bias: bool = False            # selection-only correction bias
    # speculation / sparse attention
    mtp_layers: int = 0
    indexer_heads: int = 0               # 0 = dense attention
    indexer_dim: int = 128
    indexer_topk: int = 2048
    # storage
    weight_format: str = "bf16"          # bf16 | fp8_block128 | nvfp4 | mxfp4 | exl3
    tie_embeddings: bool = False
    kv_format: str = "bf16"              # MLA cache record: bf16 (1152 bytes) | fp8_ds_mla (656 bytes; sparse attention only)

    # ---- derived -----------------------------------------------------------------
    @property
    def is_mla(self) -> bool:
        return self.attention == "mla"

    @property
    def qk_head_dim(self) -> int:
        return self.qk_nope_dim + self.qk_rope_dim if self.is_mla else self.head_dim

    @property
    def kv_record_elems(self) -> int:
        """Elements cached per token per layer (latent+rope for MLA, K and V for GQA)."""
        if self.is_mla:
            return self.kv_lora_rank + self.qk_rope_dim
        return 2 * self.num_kv_heads * self.head_dim

    @property
    def rope_dim(self) -> int:
        """Dims of a head that RoPE rotates."""
        if self.is_mla:
            return self.qk_rope_dim
        return self.rotary_dim or self.head_dim

    def window_of(self, layer: int) -> int:
        """Sliding window of ``layer`` in tokens; 0 = full causal attention."""
        if not self.sliding_window or self.is_mla:
            return 0
        if self.window_layers:
            return self.sliding_window if layer < len(self.window_layers) and self.window_layers[layer] else 0
        return self.sliding_window

    def is_moe_layer(self, layer: int) -> bool:
        return self.num_experts > 0 and layer >= self.first_dense_layers

    def attention_params(self) -> int:
        h = self.hidden
        if self.is_mla:
            q = (h * self.q_lora_rank + self.q_lora_rank * self.num_heads * self.qk_head_dim
                 if self.q_lora_rank else h * self.num_heads * self.qk_head_dim)
            kv = h * (self.kv_lora_rank + self.qk_rope_dim)
            kvb = self.kv_lora_rank * self.num_heads * (self.qk_nope_dim + self.v_head_dim)
            o = self.num_heads * self.v_head_dim * h
            return q + kv + kvb + o
        return h * (self.num_heads + 2 * self.num_kv_heads) * self.head_dim + self.num_heads * self.head_dim * h

    def expert_params(self) -> int:
        return 3 * self.hidden * self.expert_ffn

    def layer_params(self, layer: int) -> int:
        p = self.attention_params() + 2 * self.hidden
        if self.is_moe_layer(layer):
            p += self.num_experts * self.expert_params() + self.hidden * self.num_experts
            p += self.num_shared_experts * self.expert_params()
        else:
            p += 3 * self.hidden * self.dense_ffn
        return p

    def total_params(self) -> int:
        p = self.vocab_size * self.hidden * (1 if self.tie_embeddings else 2) + self.hidden
        return p + sum(self.layer_params(i) for i in range(self.num_layers))

    def to_json(self) -> str:
        return json.dumps(dataclasses.asdict(self), indent=1, sort_keys=True)

    @staticmethod
    def from_dict(d: dict[str, Any]) -> "ModelConfig":
        names = {f.name for f in dataclasses.fields(ModelConfig)}
        return ModelConfig(**{k: v for k, v in d.items() if k in names})

    def replace(self, **kw: Any) -> "ModelConfig":
        return dataclasses.replace(self, **kw)


def tiny_moe() -> ModelConfig:
    """The CPU correctness config: 2 layers, MLA, layer 0 dense, layer 1 MoE 8x top-2 + shared."""
    return ModelConfig()


def qwen3_30b_a3b() -> ModelConfig:
    """Qwen3-30B-A3B geometry (48 layers, GQA 32/4, 128 experts top-8, no shared expert)."""
    return ModelConfig(
        name="qwen3-30b-a3b", family="qwen3_moe", vocab_size=151936, num_layers=48, hidden=2048,
        attention="gqa", num_heads=32, num_kv_heads=4, head_dim=128, qk_norm=True,
        rope_theta=1.0e6, rope_interleaved=False, rms_eps=1e-6,
        dense_ffn=6144, first_dense_layers=0, num_experts=128, expert_ffn=768, top_k=8,
        scoring="softmax", num_shared_experts=0, norm_topk_prob=True, weight_format="bf16")


def deepseek_v3() -> ModelConfig:
    """DeepSeek-V3 geometry (61 layers, MLA 128 heads, 256 experts sigmoid group-limited top-8)."""
    return ModelConfig(
        name="deepseek-v3", family="deepseek_v3", vocab_size=129280, num_layers=61, hidden=7168,
        attention="mla", num_heads=128, q_lora_rank=1536, kv_lora_rank=512, qk_nope_dim=128,
        qk_rope_dim=64, v_head_dim=128, rope_theta=10000.0, rope_interleaved=True, rms_eps=1e-6,
        dense_ffn=18432, first_dense_layers=3, num_experts=256, expert_ffn=2048, top_k=8,
        scoring="sigmoid", num_groups=8, topk_groups=4, num_shared_experts=1, routed_scale=2.5,
        norm_topk_prob=True, router_bias=True, mtp_layers=1, weight_format="fp8_block128",
        # the shipped long-context setting: YaRN x40 over 4096 trained positions, mscale on the softmax scale
        rope_scaling="yarn", rope_factor=40.0, rope_original_max=4096, rope_beta_fast=32.0, rope_beta_slow=1.0,
        rope_mscale=1.0, rope_mscale_all_dim=1.0)


def deepseek_v32() -> ModelConfig:
    """DeepSeek-V3.2 geometry: V3 plus the lightning indexer and NVFP4 routed experts."""
    return deepseek_v3().replace(name="deepseek-v3.2", family="deepseek_v32", indexer_heads=64,
                                 indexer_dim=128, indexer_topk=2048, weight_format="nvfp4")


def mixtral_8x7b() -> ModelConfig:
    """Mixtral-8x7B geometry (32 layers, GQA 32/8, 8 experts top-2, softmax over the selected pair); served by the
    GQA engine, tensor names canonicalised by ``loader.families.canonical_name``."""
    return ModelConfig(
        name="mixtral-8x7b", family="qwen3_moe", vocab_size=32000, num_layers=32, hidden=4096,
        attention="gqa", num_heads=32, num_kv_heads=8, head_dim=128, qk_norm=False,
        rope_theta=1.0e6, rope_interleaved=False, rms_eps=1e-5,
        dense_ffn=14336, first_dense_layers=0, num_experts=8, expert_ffn=14336, top_k=2,
        scoring="softmax", num_shared_experts=0, norm_topk_prob=True, weight_format="bf16")


def mistral_7b() -> ModelConfig:
    """Mistral-7B-v0.1 geometry: a dense GQA 32 / 8 decoder whose every layer attends through a 4096-token sliding
    window; served by the GQA engine's dense path."""
    return ModelConfig(name="mistral-7b", family="llama", vocab_size=32000, num_layers=32, hidden=4096, attention="gqa",
                       num_heads=32, num_kv_heads=8, head_dim=128, qk_norm=False, sliding_window=4096, rope_theta=10000.0,
                       rope_interleaved=False, rms_eps=1e-5, dense_ffn=14336, first_dense_layers=32, num_experts=0,
                       expert_ffn=0, top_k=0, num_shared_experts=0)


def glm45_air() -> ModelConfig:
    """GLM-4.5-Air geometry (glm4_moe): 46 layers with one dense layer first, GQA 96 / 8 heads of 128 with biased q / k / v
    projections and RoPE on the first half of every head, 128 routed experts (FFN 1408) with sigmoid top-8 selection under a
    correction bias, one shared expert, one MTP depth."""
    return ModelConfig(name="glm-4.5-air", family="glm4_moe", vocab_size=151552, num_layers=46, hidden=4096, attention="gqa",
                       num_heads=96, num_kv_heads=8, head_dim=128, qk_norm=False, rotary_dim=64, attention_bias=True,
                       rope_theta=1.0e6, rope_interleaved=False, dense_ffn=10944, first_dense_layers=1, num_experts=128,
                       expert_ffn=1408, top_k=8, scoring="sigmoid", num_groups=1, topk_groups=1, num_shared_experts=1,
                       routed_scale=1.0, norm_topk_prob=True, router_bias=True, mtp_layers=1, rms_eps=1e-5)


def kimi_k2() -> ModelConfig:
    """Kimi-K2 geometry: the DeepSeek-V3 architecture with 64 heads and 384 routed experts (one dense layer, one
    routing group); served by the MLA engine."""
    return deepseek_v3().replace(name="kimi-k2", vocab_size=163840, num_heads=64, first_dense_layers=1, num_experts=384,
                                 num_groups=1, topk_groups=1, routed_scale=2.827, mtp_layers=0, rope_theta=50000.0,
                                 rope_factor=32.0, rope_beta_fast=1.0, rope_beta_slow=1.0)


PRESETS = {
    "tiny-moe": tiny_moe,
    "mixtral-8x7b": mixtral_8x7b,
    "mistral-7b": mistral_7b,
    "kimi-k2": kimi_k2,
    "glm-4.5-air": glm45_air,
    "qwen3-30b-a3b": qwen3_30b_a3b,
    "deepseek-v3": deepseek_v3,
    "deepseek-v3.2": deepseek_v32,
}


def scaled_down(cfg: ModelConfig, layers: int = 2, vocab: int = 2048) -> ModelConfig:
    """Same per-layer geometry with fewer layers and a small vocabulary (tests, smoke)."""
    first_dense = min(cfg.first_dense_layers, max(layers - 1, 0)) if cfg.first_dense_layers else 0
    return cfg.replace(name=cfg.name + "-mini", num_layers=layers, vocab_size=vocab,
                       first_dense_layers=first_dense)
