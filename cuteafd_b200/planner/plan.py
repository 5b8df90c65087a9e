"""``cuteafd plan``: describe a checkpoint (or a named preset) and lay it out on a box of B200s.

The report lists family, geometry, stored formats per component, hints for anything the engine
cannot serve as stored, and with a layout request the per-device memory plan, KV pool size and
expert ownership.  ``deployment()`` renders the typed launch document consumed by ``serve`` and
``expertd``.  Counterpart: rust/crates/cuteafd-loader/src/plan/mod.rs:273-1843 (PlanReport, plan,
render), plan/deployment.rs:68-109 (DeploymentSpec), plan/files.rs (role file lists).
"""
from __future__ import annotations

import hashlib
import json
import os
from collections import Counter
from dataclasses import dataclass, field

from ..config import PRESETS, ModelConfig
from ..loader import families
from ..loader.families import Hint
from . import solver


@dataclass
class PlanReport:
    model: str
    source: str                      # snapshot path or "preset"
    family: str | None
    cfg: ModelConfig
    formats: dict[str, dict[str, int]]          # role -> format -> tensor count
    stored_bytes: int
    hints: list[Hint]
    placement: solver.Placement | None = None
    request: solver.PlacementRequest | None = None
    role_files: dict[str, list[str]] = field(default_factory=dict)
    core_view: dict | None = None    # multi-core repositories: core-view, core-view-fingerprint, core-fp8-recipe

    @property
    def ready(self) -> bool:
        return not self.hints and self.family is not None and (self.placement is None or self.placement.ok)


def plan(model: str, *, layout: bool = False, fmt: str | None = None, **req_kw) -> PlanReport:
    """``model`` is a snapshot directory or a preset name (``deepseek-v3``, ``qwen3-30b-a3b`` ...)."""
    formats_by_role: dict[str, Counter] = {}
    role_files: dict[str, set] = {}
    hints: list[Hint] = []
    stored = 0
    view = None
    if model in PRESETS and not os.path.exists(model):
        cfg = PRESETS[model]()
        if fmt:
            cfg = cfg.replace(weight_format=fmt)
        fam = next((f for f in families.REGISTRY if f.id == cfg.family), None)
        source = "preset"
        comp = solver.component_bytes(cfg, solver.PlacementRequest(cfg))
        stored = sum(v for k, v in comp.items() if k not in ("one_expert_all_layers", "mtp")) + comp["mtp"]
        formats_by_role = {"routed_expert": Counter({cfg.weight_format: cfg.num_experts * 3}),
                           "attention": Counter({"bf16" if cfg.weight_format != "fp8_block128" else "fp8_block128": 1})}
    else:
        from ..loader.load import open_snapshot
        snap = open_snapshot(model)
        cfg, fam, source = snap.cfg, snap.family, snap.path
        if fmt:
            cfg = cfg.replace(weight_format=fmt)
        hints = snap.hints()
        view = snap.view.settings() if snap.view is not None else None
        for op in snap.operands.values():
            role = snap.model.classify(op.weight)[0] if snap.model else "other"
            formats_by_role.setdefault(role, Counter())[op.format] += 1
            stored += op.stored_bytes(snap.catalog)
            role_files.setdefault(role, set()).add(os.path.basename(snap.catalog.entries[op.weight].file))
    rep = PlanReport(cfg.name, source, fam.id if fam else None, cfg, {r: dict(c) for r, c in formats_by_role.items()},
                     stored, hints, role_files={r: sorted(f) for r, f in role_files.items()}, core_view=view)
    if layout:
        pool_bytes = req_kw.pop("kv_pool_bytes", None)
        if pool_bytes and req_kw.get("pool_tokens_target") is None:
            # a pool given in bytes (the reference's KV_POOL_SIZE): tokens of this model's cache record that fit in it
            per_token = solver.kv_bytes_per_token_per_layer(cfg, req_kw.get("kv_format") or "auto") * cfg.num_layers
            req_kw["pool_tokens_target"] = max(64, int(pool_bytes) // per_token // 64 * 64)
        rep.request = solver.PlacementRequest(cfg, **{k: v for k, v in req_kw.items() if v is not None})
        rep.placement = solver.solve(rep.request)
    return rep


def _gib(n: float) -> str:
    return f"{n / solver.GIB:8.2f} GiB"


def render(rep: PlanReport) -> str:
    c = rep.cfg
    L = [f"model      {rep.model}   ({rep.source})",
         f"family     {rep.family or 'UNKNOWN'}",
         f"geometry   {c.num_layers} layers, hidden {c.hidden}, vocab {c.vocab_size}, "
         + (f"MLA {c.num_heads} heads (q_lora {c.q_lora_rank}, kv_lora {c.kv_lora_rank}, nope {c.qk_nope_dim}, rope {c.qk_rope_dim}, v {c.v_head_dim})"
            if c.is_mla else f"GQA {c.num_heads}/{c.num_kv_heads} heads x {c.head_dim}"),
         f"ffn        dense {c.dense_ffn} x {c.first_dense_layers} layers; {c.num_experts} routed experts x {c.expert_ffn} "
         f"({c.scoring} top-{c.top_k}" + (f", {c.num_groups} groups keep {c.topk_groups}" if c.num_groups > 1 else "") + ")"
         + (f" + {c.num_shared_experts} shared" if c.num_shared_experts else ""),
         f"extras     mtp layers {c.mtp_layers}; indexer " + (f"{c.indexer_heads} heads x {c.indexer_dim}, top-{c.indexer_topk}" if c.indexer_heads else "none"),
         f"stored     {_gib(rep.stored_bytes)}   parameters {c.total_params()/1e9:.1f} B"]
    for role, f in sorted(rep.formats.items()):
        L.append(f"  {role:<15} " + ", ".join(f"{k} x{v}" for k, v in sorted(f.items())))
    if rep.core_view:
        L.append(f"core view  {rep.core_view['core-view']} (fingerprint {rep.core_view['core-view-fingerprint'][:16]})"
                 + (f", encoded at load: {rep.core_view['core-fp8-recipe']}" if rep.core_view.get("core-fp8-recipe") else ""))
    if rep.hints:
        L.append(f"hints      {len(rep.hints)} operand(s) cannot be served as stored:")
        for h in rep.hints[:20]:
            L.append(f"  - {h.what}\n      -> {h.how}")
    else:
        L.append("hints      none: every operand has a kernel path")
    p = rep.placement
    if p is not None:
        L.append("")
        if not p.ok:
            L.append(f"layout     REJECTED: {p.reason}")
        else:
            L.append(f"layout     {p.layout}; speculator {p.speculator}; decode lanes {p.decode_lanes}")
            L.append(f"kv pool    {p.kv_pool_tokens} tokens x {p.kv_bytes_per_token} B/token/device "
                     f"({p.max_concurrency_at_context} sequences at full context)")
            for g in p.devices:
                if g.role == "idle":
                    continue
                cats = g.by_category()
                L.append(f"  gpu{g.index} {g.role:<17} used {_gib(g.used)} free {_gib(g.free)} | "
                         + " ".join(f"{k} {v/solver.GIB:.1f}" for k, v in cats.items() if v))
            if p.expert_ranges:
                if p.expert_ranks == 0 and p.attention_ranks > 1:
                    L.append(f"experts    [0:{p.expert_ranges[-1][1]}) on every rank of the tensor-parallel group")
                else:
                    L.append("experts    " + " ".join(f"[{lo}:{hi})" for lo, hi in p.expert_ranges))
            for n in p.notes:
                L.append(f"note       {n}")
    L.append(f"ready      {'yes' if rep.ready else 'no'}")
    return "\n".join(L)


def to_json(rep: PlanReport) -> dict:
    import dataclasses
    return {"model": rep.model, "source": rep.source, "family": rep.family, "config": dataclasses.asdict(rep.cfg),
            "formats": rep.formats, "stored_bytes": rep.stored_bytes,
            "hints": [{"what": h.what, "how": h.how} for h in rep.hints],
            "placement": rep.placement.to_json() if rep.placement else None, "ready": rep.ready,
            "core_view": rep.core_view}


def deployment(rep: PlanReport, master_addr: str = "127.0.0.1", master_port: int = 29500) -> dict:
    """Typed launch document: one entry per rank with its role, device, expert range and budgets."""
    p = rep.placement
    if p is None or not p.ok:
        raise ValueError("a deployment needs an accepted layout (plan with layout=True)")
    ranks = []
    n_att = p.attention_ranks * p.pipeline_stages
    for i in range(n_att + p.expert_ranks):
        g = p.devices[i]
        entry = {"rank": i, "device": g.index, "role": g.role, "memory": g.by_category(), "free_bytes": g.free}
        if i < n_att:
            entry.update(tp_rank=i % p.attention_ranks, pp_stage=i // p.attention_ranks)
            if p.expert_ranks == 0 and p.expert_ranges and p.attention_ranks == 1:
                entry["experts"] = list(p.expert_ranges[i])          # (a tensor-parallel group keeps every expert on every rank)
        else:
            entry["experts"] = list(p.expert_ranges[i - n_att])
        ranks.append(entry)
    body = {"model": rep.model, "source": rep.source, "family": rep.family, "layout": p.layout,
            "world_size": len(ranks), "attention_ranks": p.attention_ranks, "expert_ranks": p.expert_ranks,
            "pipeline_stages": p.pipeline_stages, "engine": p.engine, "kv_pool_tokens": p.kv_pool_tokens, "speculator": p.speculator,
            "decode_lanes": p.decode_lanes, "prefill_rows": rep.request.prefill_rows, "decode_rows": rep.request.decode_rows,
            "max_context_tokens": rep.request.max_context_tokens, "rendezvous": {"master_addr": master_addr, "master_port": master_port},
            "ranks": ranks}
    body["plan_hash"] = hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()[:16]
    return body
