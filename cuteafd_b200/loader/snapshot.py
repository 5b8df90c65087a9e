"""Hugging Face snapshot layout: ``config.json`` <-> ``ModelConfig``, snapshot resolution, and
writers of random-init snapshots in each shipped weight format.

A snapshot is a directory with config.json, model.safetensors.index.json and shards; runs load it
"as shipped", nothing is repacked on disk.  Counterpart: rust/crates/cuteafd-loader/src/snapshot.rs
(resolve), plan/testing.rs (snapshot writers for tests).
"""
from __future__ import annotations

import json
import os

import torch

from ..config import ModelConfig
from ..ref.model import init_weights
from . import formats
from .safetensors_io import write_sharded

ARCH = {"llama": "LlamaForCausalLM", "qwen3_moe": "Qwen3MoeForCausalLM", "deepseek_v3": "DeepseekV3ForCausalLM",
        "deepseek_v32": "DeepseekV32ForCausalLM", "tiny_moe": "DeepseekV3ForCausalLM", "glm4_moe": "Glm4MoeForCausalLM",
        "qwen2": "Qwen2ForCausalLM"}


def to_hf_config(cfg: ModelConfig) -> dict:
    d = {"architectures": [ARCH.get(cfg.family, "DeepseekV3ForCausalLM")], "model_type": cfg.family,
         "vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden, "num_hidden_layers": cfg.num_layers,
         "num_attention_heads": cfg.num_heads, "rms_norm_eps": cfg.rms_eps, "rope_theta": cfg.rope_theta,
         "tie_word_embeddings": cfg.tie_embeddings, "torch_dtype": "bfloat16",
         "intermediate_size": cfg.dense_ffn, "moe_intermediate_size": cfg.expert_ffn,
         "num_experts_per_tok": cfg.top_k, "norm_topk_prob": cfg.norm_topk_prob,
         "cuteafd": {"name": cfg.name, "rope_interleaved": cfg.rope_interleaved, "family": cfg.family}}
    if cfg.is_mla:
        d.update(q_lora_rank=cfg.q_lora_rank or None, kv_lora_rank=cfg.kv_lora_rank, qk_nope_head_dim=cfg.qk_nope_dim,
                 qk_rope_head_dim=cfg.qk_rope_dim, v_head_dim=cfg.v_head_dim, n_routed_experts=cfg.num_experts,
                 n_shared_experts=cfg.num_shared_experts, first_k_dense_replace=cfg.first_dense_layers,
                 scoring_func=cfg.scoring, n_group=cfg.num_groups, topk_group=cfg.topk_groups,
                 routed_scaling_factor=cfg.routed_scale, num_nextn_predict_layers=cfg.mtp_layers,
                 topk_method="noaux_tc" if cfg.router_bias else "greedy")
        if cfg.indexer_heads:
            d.update(index_n_heads=cfg.indexer_heads, index_head_dim=cfg.indexer_dim, index_topk=cfg.indexer_topk)
    elif cfg.family == "glm4_moe":
        d.update(num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, n_routed_experts=cfg.num_experts,
                 n_shared_experts=cfg.num_shared_experts, first_k_dense_replace=cfg.first_dense_layers, n_group=cfg.num_groups,
                 topk_group=cfg.topk_groups, routed_scaling_factor=cfg.routed_scale, use_qk_norm=cfg.qk_norm,
                 attention_bias=cfg.attention_bias, partial_rotary_factor=cfg.rope_dim / cfg.head_dim,
                 num_nextn_predict_layers=cfg.mtp_layers)
    else:
        d.update(num_key_value_heads=cfg.num_kv_heads, head_dim=cfg.head_dim, num_experts=cfg.num_experts,
                 decoder_sparse_step=1, mlp_only_layers=list(range(cfg.first_dense_layers)), qk_norm=cfg.qk_norm)
        if cfg.attention_bias:
            d["attention_bias"] = True
    if cfg.sliding_window and not cfg.is_mla:
        d.update(sliding_window=cfg.sliding_window, use_sliding_window=True,
                 layer_types=["sliding_attention" if cfg.window_of(i) else "full_attention" for i in range(cfg.num_layers)])
    if cfg.rope_scaling != "none":
        rs = {"type": cfg.rope_scaling, "rope_type": cfg.rope_scaling, "factor": cfg.rope_factor,
              "original_max_position_embeddings": cfg.rope_original_max}
        if cfg.rope_scaling == "yarn":
            rs.update(beta_fast=cfg.rope_beta_fast, beta_slow=cfg.rope_beta_slow, mscale=cfg.rope_mscale,
                      mscale_all_dim=cfg.rope_mscale_all_dim)
        if cfg.rope_scaling == "llama3":
            rs.update(low_freq_factor=cfg.rope_low_freq_factor, high_freq_factor=cfg.rope_high_freq_factor)
        d["rope_scaling"] = rs
    if cfg.weight_format == "fp8_block128":
        d["quantization_config"] = {"quant_method": "fp8", "fmt": "e4m3", "weight_block_size": [128, 128],
                                    "activation_scheme": "dynamic"}
    elif cfg.weight_format == "nvfp4":
        d["quantization_config"] = {"quant_method": "modelopt", "quant_algo": "NVFP4", "group_size": 16}
    elif cfg.weight_format == "mxfp4":
        d["quantization_config"] = {"quant_method": "mxfp4", "group_size": 32}
    elif cfg.weight_format.startswith("exl3"):
        d["quantization_config"] = {"quant_method": "exl3", "bits": 4}
    return d


def _windows(d: dict) -> dict:
    """config.json sliding-window fields -> ModelConfig fields.  ``layer_types`` names the windowed layers where it is
    present; the Qwen2 / Qwen3 form (``use_sliding_window`` with ``max_window_layers``) windows the layers from that
    index on; a bare ``sliding_window`` (Mistral, Mixtral) windows every layer."""
    w, n = d.get("sliding_window"), d["num_hidden_layers"]
    kinds = d.get("layer_types")
    if kinds:
        unknown = set(kinds) - {"sliding_attention", "full_attention"}
        if unknown or len(kinds) != n:
            raise ValueError(f"layer_types {sorted(unknown)} / {len(kinds)} entries for {n} layers is not supported")
        flags = tuple(1 if k == "sliding_attention" else 0 for k in kinds)
    elif str(d.get("model_type", "")).startswith("qwen"):
        first = d.get("max_window_layers", n) if d.get("use_sliding_window") else n
        flags = tuple(1 if i >= first else 0 for i in range(n))
    else:
        flags = (1,) * n
    if not w or not any(flags):
        return {}
    return {"sliding_window": int(w), "window_layers": () if all(flags) else flags}


def _rope_scaling(d: dict) -> dict:
    """config.json ``rope_scaling`` / ``rope_parameters`` -> ModelConfig fields.  Unknown kinds are refused: serving a
    long-context checkpoint with the wrong frequencies gives fluent nonsense, not an error."""
    rs = d.get("rope_scaling") or d.get("rope_parameters") or {}
    kind = rs.get("rope_type") or rs.get("type") or "none"
    if kind in ("none", "default") or not rs:
        return {}
    if kind not in ("linear", "llama3", "yarn"):
        raise ValueError(f"unsupported rope scaling {kind!r}")
    out = dict(rope_scaling=kind, rope_factor=float(rs.get("factor", 1.0)),
               rope_original_max=int(rs.get("original_max_position_embeddings") or d.get("max_position_embeddings") or 4096))
    if kind == "yarn":
        out.update(rope_beta_fast=float(rs.get("beta_fast") or 32.0), rope_beta_slow=float(rs.get("beta_slow") or 1.0),
                   rope_mscale=float(rs.get("mscale") or 1.0), rope_mscale_all_dim=float(rs.get("mscale_all_dim") or 0.0))
    if kind == "llama3":
        out.update(rope_low_freq_factor=float(rs.get("low_freq_factor", 1.0)), rope_high_freq_factor=float(rs.get("high_freq_factor", 4.0)))
    return out


def from_hf_config(d: dict) -> ModelConfig:
    """Map a config.json onto the engine's geometry.  Unknown architectures raise ValueError."""
    mt = d.get("model_type", "")
    extra = d.get("cuteafd", {})
    q = d.get("quantization_config") or {}
    fmt = {"fp8": "fp8_block128", "modelopt": "nvfp4", "mxfp4": "mxfp4", "exl3": "exl3"}.get(q.get("quant_method", ""), "bf16")
    common = dict(name=extra.get("name", d.get("_name_or_path", mt) or mt), vocab_size=d["vocab_size"],
                  num_layers=d["num_hidden_layers"], hidden=d["hidden_size"], num_heads=d["num_attention_heads"],
                  rms_eps=d.get("rms_norm_eps", 1e-6), rope_theta=float(d.get("rope_theta") or (d.get("rope_parameters") or {}).get("rope_theta") or 10000.0),
                  tie_embeddings=bool(d.get("tie_word_embeddings", False)), dense_ffn=d.get("intermediate_size", 0),
                  expert_ffn=d.get("moe_intermediate_size", 0), top_k=d.get("num_experts_per_tok", 0),
                  norm_topk_prob=bool(d.get("norm_topk_prob", True)), weight_format=fmt, **_rope_scaling(d))
    if mt in ("deepseek_v3", "deepseek_v32", "deepseek_v2", "tiny_moe", "glm_moe_dsa", "kimi_k2"):
        return ModelConfig(
            family=extra.get("family", "deepseek_v32" if d.get("index_n_heads") else "deepseek_v3"), attention="mla",
            q_lora_rank=d.get("q_lora_rank") or 0, kv_lora_rank=d["kv_lora_rank"], qk_nope_dim=d["qk_nope_head_dim"],
            qk_rope_dim=d["qk_rope_head_dim"], v_head_dim=d["v_head_dim"],
            rope_interleaved=extra.get("rope_interleaved", True), first_dense_layers=d.get("first_k_dense_replace", 0),
            num_experts=d.get("n_routed_experts", 0), scoring=d.get("scoring_func", "softmax"),
            num_groups=d.get("n_group", 1) or 1, topk_groups=d.get("topk_group", 1) or 1,
            num_shared_experts=d.get("n_shared_experts", 0) or 0, routed_scale=d.get("routed_scaling_factor", 1.0),
            router_bias=d.get("topk_method") == "noaux_tc", mtp_layers=d.get("num_nextn_predict_layers", 0) or 0,
            indexer_heads=d.get("index_n_heads", 0) or 0, indexer_dim=d.get("index_head_dim", 128),
            indexer_topk=d.get("index_topk", 2048), **common)
    if mt in ("qwen3_moe", "qwen3", "qwen2_moe", "mixtral"):
        # refuse what the engines would silently compute differently
        if d.get("shared_expert_intermediate_size"):
            raise ValueError("a gated shared expert (shared_expert_intermediate_size) is not supported")
        if d.get("decoder_sparse_step", 1) not in (0, 1):
            raise ValueError("interleaved dense / sparse layers (decoder_sparse_step > 1) are not supported")
        dense_layers = sorted(d.get("mlp_only_layers", []) or [])
        if dense_layers != list(range(len(dense_layers))):
            raise ValueError("dense layers must be the first layers of the stack")
        if d.get("attention_bias"):
            raise ValueError("projection biases are not supported for this model type")
        return ModelConfig(
            family="qwen3_moe", attention="gqa", num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim", d["hidden_size"] // d["num_attention_heads"]), qk_norm=bool(d.get("qk_norm", mt.startswith("qwen3"))),
            rope_interleaved=extra.get("rope_interleaved", False), first_dense_layers=len(d.get("mlp_only_layers", []) or []),
            num_experts=d.get("num_experts", d.get("num_local_experts", 0)), scoring="softmax", num_shared_experts=0, **_windows(d), **common)
    if mt == "glm4_moe":
        # GLM-4.5 / 4.6: GQA with biased q / k / v projections and RoPE on part of every head, sigmoid routing under a
        # correction bias (noaux_tc), one shared expert, dense layers first, optional MTP depth
        hd = d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"]
        rot = int(round(hd * float(d.get("partial_rotary_factor", 1.0))))
        if hd != 128 or rot not in (64, 128):
            raise ValueError(f"glm4_moe with head_dim {hd} and {rot} rotated dims is not supported (128 with 64 or 128)")
        return ModelConfig(
            family="glm4_moe", attention="gqa", num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]), head_dim=hd,
            qk_norm=bool(d.get("use_qk_norm", False)), rotary_dim=0 if rot == hd else rot, attention_bias=bool(d.get("attention_bias", False)),
            rope_interleaved=extra.get("rope_interleaved", False), first_dense_layers=d.get("first_k_dense_replace", 0),
            num_experts=d.get("n_routed_experts", 0), scoring="sigmoid", num_groups=d.get("n_group", 1) or 1,
            topk_groups=d.get("topk_group", 1) or 1, num_shared_experts=d.get("n_shared_experts", 0) or 0,
            routed_scale=d.get("routed_scaling_factor", 1.0), router_bias=True, mtp_layers=d.get("num_nextn_predict_layers", 0) or 0,
            **common)
    if mt == "qwen2":
        # dense Qwen2 / Qwen2.5: a Llama-shaped stack whose q / k / v projections carry a bias
        return ModelConfig(
            family="qwen2", attention="gqa", num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"], qk_norm=False, attention_bias=True,
            rope_interleaved=extra.get("rope_interleaved", False), first_dense_layers=d["num_hidden_layers"], num_experts=0,
            num_shared_experts=0, **_windows(d), **dict(common, top_k=0, expert_ffn=0))
    if mt in ("llama", "mistral"):
        # dense GQA decoders without projection biases: every layer takes the dense SwiGLU path
        if d.get("attention_bias") or d.get("mlp_bias"):
            raise ValueError("projection biases are not supported")
        return ModelConfig(
            family="llama", attention="gqa", num_kv_heads=d.get("num_key_value_heads", d["num_attention_heads"]),
            head_dim=d.get("head_dim") or d["hidden_size"] // d["num_attention_heads"], qk_norm=False,
            rope_interleaved=extra.get("rope_interleaved", False), first_dense_layers=d["num_hidden_layers"], num_experts=0,
            num_shared_experts=0, **_windows(d), **dict(common, top_k=0, expert_ffn=0))
    raise ValueError(f"unsupported model_type {mt!r}")


def resolve(path: str) -> str:
    """Accept a snapshot directory or a hub cache root (models--org--name/snapshots/<rev>)."""
    if os.path.isfile(os.path.join(path, "config.json")):
        return path
    snaps = os.path.join(path, "snapshots")
    if os.path.isdir(snaps):
        revs = sorted(os.listdir(snaps))
        if revs:
            return os.path.join(snaps, revs[-1])
    raise FileNotFoundError(f"{path}: no config.json and no snapshots/ directory")


def core_view(path: str, view: str | None = None):
    """The verified core view of a multi-core repository (``loader/mc.py``), or None for a plain checkpoint served as
    it is.  ``view`` None reads ``$CUTEAFD_CORE_VIEW`` (what ``serve --core-view`` sets), default ``original``."""
    from . import mc
    view = view or os.environ.get("CUTEAFD_CORE_VIEW", "") or "original"
    return mc.select(mc.discover(resolve(path)), view)


def view_weight_map(path: str, view: str | None = None) -> dict[str, str] | None:
    """tensor name -> shard of the selected view; None when the directory is a plain checkpoint (every shard belongs)."""
    sel = core_view(path, view)
    if sel is None:
        return None
    with open(os.path.join(resolve(path), sel.view.index)) as f:
        return json.load(f)["weight_map"]


def read_config(path: str, view: str | None = None) -> tuple[ModelConfig, dict]:
    sel = core_view(path, view)
    with open(os.path.join(resolve(path), sel.view.config if sel is not None else "config.json")) as f:
        d = json.load(f)
    return from_hf_config(d), d


def _quantised(name: str, cfg: ModelConfig, scope: str) -> bool:
    if not name.endswith(".weight") or "norm" in name or "embed_tokens" in name or name.startswith("lm_head"):
        return False
    if ".mlp.gate.weight" in name:
        return False
    if scope == "experts":
        return ".mlp.experts." in name
    return ".mlp." in name or ".self_attn." in name


def write_random_snapshot(cfg: ModelConfig, directory: str, fmt: str | None = None, seed: int = 0,
                          scope: str = "experts", shard_bytes: int = 1 << 30) -> str:
    """Random-init snapshot of ``cfg`` in format ``fmt`` (bf16 | fp8_block128 | nvfp4 | mxfp4 | exl3_k4).

    ``scope`` = "experts": only routed experts carry the quantised format (the usual shipped
    mix); "linear": every projection does (DeepSeek FP8 style)."""
    fmt = fmt or cfg.weight_format
    cfg = cfg.replace(weight_format=fmt if not fmt.startswith("exl3") else "exl3")
    params = init_weights(cfg, seed=seed)
    gen = torch.Generator().manual_seed(seed + 17)
    out: dict[str, torch.Tensor] = {}
    for name, t in params.items():
        if fmt != "bf16" and _quantised(name, cfg, scope) and t.shape[-1] % 128 == 0 and t.shape[0] % 16 == 0:
            out.update(formats.encode(t, fmt, name[: -len(".weight")], gen))
        elif name.endswith("e_score_correction_bias"):
            out[name] = t.float()
        else:
            out[name] = t.to(torch.bfloat16)
    os.makedirs(directory, exist_ok=True)
    with open(os.path.join(directory, "config.json"), "w") as f:
        json.dump(to_hf_config(cfg), f, indent=1, sort_keys=True)
    write_sharded(directory, out, shard_bytes)
    return directory
