"""Serving capacity tables: the sizes a deployment is built around, derived instead of hand-kept.

* ``prefill_unit_rows(top_k)``   rows of one prefill unit such that the rows it dispatches to the experts
                                 (rows x top_k) stay within ``RESERVE_ROWS`` per exchange step; whole 64-row pages.
* ``prefill_waves(rows, unit)``  how a prompt is cut into units (all full but the last, which is padded up to 64).
* ``default_prewarm(...)``       decode step geometries worth capturing as CUDA graphs before traffic arrives, for a
                                 server that has no trace of an earlier run: plain decode at every batch size up to
                                 the concurrency, and the verify shapes of a draft block (every sequence carrying the
                                 same number of drafts, which is what a settled history policy produces).
* ``workspace_bytes(cfg, rows)`` activation workspaces of one engine step of ``rows`` tokens (what the planner charges
                                 per GPU next to weights and KV).

Counterpart: rust/crates/cuteafd-loader/src/serving_capacity/prefill_waves.rs:10-36 (RESERVE_ROWS, unit rows per
top-k), ``*_graphs.rs`` / ``*_prewarm.json`` (graph prewarm lists).  The reference ships measured tables per family
and host; here they follow from the model geometry.
"""
from __future__ import annotations

from ..config import ModelConfig

RESERVE_ROWS = 8192
PIPELINE_DEPTH = 3              # exchange waves in flight (transfer in, expert GEMMs, transfer out)
PAGE = 64


def prefill_unit_rows(top_k: int, reserve_rows: int = RESERVE_ROWS) -> int:
    k = max(1, top_k)
    return max(PAGE, reserve_rows // k // PAGE * PAGE)


def prefill_waves(rows: int, unit: int) -> list[int]:
    """Unit sizes for a prompt of ``rows`` tokens."""
    out = [unit] * (rows // unit)
    rest = rows % unit
    if rest:
        out.append((rest + PAGE - 1) // PAGE * PAGE)
    return out


def default_prewarm(concurrency: int, draft_block: int = 0, limit: int = 48) -> list[list[int]]:
    """[sequences, rows, longest run] triples, most useful first, at most ``limit``."""
    sizes = sorted({1, 2, 4, 8, 16, 32, 64, concurrency} | set(range(1, min(concurrency, 8) + 1)))
    sizes = [s for s in sizes if s <= concurrency]
    keys = [[s, s, 1] for s in sizes]
    if draft_block > 0:
        for s in sizes:
            for d in (draft_block, 1):                       # a full block, and the one-draft shape of a cautious policy
                keys.append([s, s * (1 + d), 1 + d])
    seen, out = set(), []
    for k in keys:
        if tuple(k) not in seen:
            seen.add(tuple(k))
            out.append(k)
    return out[:limit]


def workspace_bytes(cfg: ModelConfig, rows: int) -> int:
    """bf16 activation slabs of one step: residual, qkv / latent projections, attention out, router logits, FFN
    intermediates, and the MoE exchange rows (rows x top_k, in and out)."""
    h = cfg.hidden
    if cfg.is_mla:
        attn = (cfg.q_lora_rank + cfg.kv_lora_rank + cfg.qk_rope_dim) + cfg.num_heads * (cfg.qk_head_dim + cfg.v_head_dim + cfg.kv_lora_rank + cfg.qk_rope_dim)
    else:
        attn = (cfg.num_heads * 2 + cfg.num_kv_heads * 2) * cfg.head_dim
    ffn = max(cfg.dense_ffn if cfg.first_dense_layers or not cfg.num_experts else 0, cfg.expert_ffn * max(cfg.num_shared_experts, 0)) * 2
    moe = cfg.top_k * (2 * h + 2 * cfg.expert_ffn) if cfg.num_experts else 0
    per_row = 2 * (3 * h + attn + ffn + moe) + 4 * max(cfg.num_experts, 1)
    return rows * per_row
