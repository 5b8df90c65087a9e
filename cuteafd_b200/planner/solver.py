"""One CPU-only placement solver shared by ``cuteafd plan`` and runtime admission.

Input: a model geometry with per-component byte sizes, an inventory of GPUs, and a layout request
(attention tensor-parallel degree, expert-parallel ranks, pipeline stages, or "auto").  Output: a
per-device memory layout made of typed demands, the KV pool size, expert ownership per rank, and
capacity facts (concurrency, context).  Order of allocation is pool-first: fixed weights and
workspaces are placed, then the KV pool takes what is left up to its target, and the plan is
rejected only if the pool cannot reach its minimum.

Counterpart: rust/crates/cuteafd-loader/src/placement/mod.rs:70-330 (PlacementRequest, Inventory,
GpuBudget, Baseline, LayerDemand, LayerMode), placement/solve.rs:85-229, pool.rs, reserve.rs,
graph_reserve.rs.  The reference places attention on 1-2 GPUs and expert *slices* on up to 8 remote
boxes; here every rank is a B200 of one NVLink domain and experts are partitioned by id.
"""
from __future__ import annotations

import math
from dataclasses import asdict, dataclass, field

from ..config import ModelConfig

GIB = 1 << 30
B200_HBM_BYTES = 183_359 * (1 << 20)          # what nvidia-smi reports for a 180 GB part
BITS = {"bf16": 16.0, "fp8_block128": 8.0 + 32.0 / (128 * 128), "nvfp4": 4.0 + 8.0 / 16, "mxfp4": 4.0 + 8.0 / 32,
        "exl3": 4.0, "exl3_k2": 2.0, "exl3_k3": 3.0, "exl3_k4": 4.0, "exl3_k6": 6.0, "exl3_k8": 8.0}
CATEGORIES = ("weights", "experts", "kv_pool", "workspace", "exchange", "graphs", "reserve")


@dataclass
class Demand:
    category: str
    owner: str
    bytes: int


@dataclass
class GpuBudget:
    index: int
    capacity: int
    role: str = "idle"                      # "attention" | "expert" | "attention+expert" | "idle"
    demands: list[Demand] = field(default_factory=list)

    @property
    def used(self) -> int:
        return sum(d.bytes for d in self.demands)

    @property
    def free(self) -> int:
        return self.capacity - self.used

    def add(self, category: str, owner: str, nbytes: int) -> None:
        if nbytes > 0:
            self.demands.append(Demand(category, owner, int(nbytes)))

    def by_category(self) -> dict[str, int]:
        out = {c: 0 for c in CATEGORIES}
        for d in self.demands:
            out[d.category] = out.get(d.category, 0) + d.bytes
        return out


@dataclass
class PlacementRequest:
    cfg: ModelConfig
    gpus: int = 8
    gpu_memory_cap: int = B200_HBM_BYTES
    attention_ranks: int | None = None      # tensor-parallel degree of the backbone; None = auto
    expert_ranks: int | None = None         # expert-parallel ranks; 0 = experts share the attention GPUs
    pipeline_stages: int = 1
    pool_tokens_target: int = 2_097_152     # reference default KV pool target (2M tokens), min 256K
    pool_tokens_min: int = 262_144
    max_context_tokens: int = 131_072
    concurrency: int = 32
    prefill_rows: int = 8192
    decode_rows: int = 64
    decode_lanes: int = 1
    speculator: str = "auto"                # auto | off | mtp
    expert_format: str | None = None        # override of cfg.weight_format for routed experts
    backbone_format: str | None = None      # attention / dense / shared weights (default bf16, fp8 for fp8 checkpoints)
    kv_format: str = "auto"                 # auto | bf16 | fp8_ds_mla
    reserve_fraction: float = 0.04          # allocator slack + CUDA context per device
    redundant_experts: int = 0              # extra hot-expert replicas per expert rank
    # Decode-graph arena per attention device.  None = the unmeasured default (256 MiB per lane); a measured value is
    # base + extra bytes from a prewarm file a serving run wrote (``EngineBackend.save_prewarm``), or a user override.
    graph_reserve_bytes: int | None = None
    graph_reserve_source: str = "default"


@dataclass
class Placement:
    ok: bool
    reason: str
    layout: str
    attention_ranks: int
    expert_ranks: int
    pipeline_stages: int
    devices: list[GpuBudget]
    expert_ranges: list[tuple[int, int]]
    kv_pool_tokens: int
    kv_bytes_per_token: int
    max_concurrency_at_context: int
    speculator: str
    decode_lanes: int
    notes: list[str] = field(default_factory=list)
    score: float = 0.0
    engine: str = ""                   # which engine serves this layout today ("" = none yet, see the last note)

    def to_json(self) -> dict:
        d = asdict(self)
        for dev, g in zip(d["devices"], self.devices):
            dev["used"], dev["free"], dev["by_category"] = g.used, g.free, g.by_category()
        return d


def weight_bytes(params: int, fmt: str) -> int:
    return int(math.ceil(params * BITS.get(fmt, 16.0) / 8.0))


def kv_bytes_per_token_per_layer(cfg: ModelConfig, kv_format: str) -> int:
    if cfg.is_mla:
        if kv_format in ("auto", "fp8_ds_mla") and cfg.weight_format != "bf16":
            return cfg.kv_lora_rank + 4 * (cfg.kv_lora_rank // 128) + 2 * cfg.qk_rope_dim      # 656 B for 512 + 64
        return 2 * (cfg.kv_lora_rank + cfg.qk_rope_dim)
    return 2 * 2 * cfg.num_kv_heads * cfg.head_dim


def component_bytes(cfg: ModelConfig, req: PlacementRequest) -> dict[str, int]:
    """Bytes of every component of the whole model (before sharding)."""
    efmt = req.expert_format or cfg.weight_format
    bfmt = req.backbone_format or ("fp8_block128" if cfg.weight_format == "fp8_block128" else "bf16")
    n_moe = sum(1 for i in range(cfg.num_layers) if cfg.is_moe_layer(i))
    n_dense = cfg.num_layers - n_moe
    out = {
        "embedding": cfg.vocab_size * cfg.hidden * 2,
        "head": 0 if cfg.tie_embeddings else cfg.vocab_size * cfg.hidden * 2,
        "attention": cfg.num_layers * weight_bytes(cfg.attention_params(), bfmt),
        "dense_ffn": n_dense * weight_bytes(3 * cfg.hidden * cfg.dense_ffn, bfmt),
        "shared_experts": n_moe * cfg.num_shared_experts * weight_bytes(cfg.expert_params(), bfmt),
        "router": n_moe * cfg.hidden * cfg.num_experts * 2,
        "norms": (2 * cfg.num_layers + 1) * cfg.hidden * 2,
        "routed_experts": n_moe * cfg.num_experts * weight_bytes(cfg.expert_params(), efmt),
        "one_expert_all_layers": n_moe * weight_bytes(cfg.expert_params(), efmt),
        "indexer": cfg.num_layers * weight_bytes(cfg.hidden * (cfg.indexer_heads * cfg.indexer_dim + cfg.indexer_dim + cfg.indexer_heads), bfmt)
        if cfg.indexer_heads else 0,
        "mtp": cfg.mtp_layers * (weight_bytes(cfg.attention_params() + 2 * cfg.hidden * cfg.hidden, bfmt)
                                 + cfg.num_experts * weight_bytes(cfg.expert_params(), efmt)),
    }
    return out


def _expert_ranges(n: int, ranks: int) -> list[tuple[int, int]]:
    base, rem = divmod(n, ranks)
    out, lo = [], 0
    for r in range(ranks):
        hi = lo + base + (1 if r < rem else 0)
        out.append((lo, hi))
        lo = hi
    return out


def _place(req: PlacementRequest, att: int, exp: int, pp: int) -> Placement:
    cfg = req.cfg
    comp = component_bytes(cfg, req)
    colocated = exp == 0
    n_dev = att * pp + exp
    devices = [GpuBudget(i, req.gpu_memory_cap) for i in range(req.gpus)]
    notes: list[str] = []
    if n_dev > req.gpus:
        return Placement(False, f"layout needs {n_dev} GPUs, inventory has {req.gpus}", "", att, exp, pp, devices, [], 0, 0, 0,
                         "off", req.decode_lanes)
    spec = req.speculator
    if spec == "auto":
        spec = "mtp" if cfg.mtp_layers else "off"
    if spec == "mtp" and not cfg.mtp_layers:
        return Placement(False, "speculator mtp requested but the checkpoint has no MTP layers", "", att, exp, pp, devices, [], 0, 0, 0,
                         "off", req.decode_lanes)
    kv_tok_layer = kv_bytes_per_token_per_layer(cfg, req.kv_format)
    layers_per_stage = math.ceil(cfg.num_layers / pp)
    # MLA latent KV is replicated across attention TP ranks; GQA KV heads are split when they divide.
    kv_shard = 1 if cfg.is_mla else min(att, cfg.num_kv_heads)
    kv_per_token_dev = kv_tok_layer * layers_per_stage // kv_shard
    act_rows = max(req.prefill_rows, req.decode_rows)
    ranges = _expert_ranges(cfg.num_experts, exp if exp else att * pp) if cfg.num_experts else []
    e_max = max((hi - lo for lo, hi in ranges), default=0)
    # ---- attention devices ---------------------------------------------------------------------------
    for s in range(pp):
        for t in range(att):
            g = devices[s * att + t]
            g.role = "attention+expert" if colocated else "attention"
            frac = layers_per_stage / cfg.num_layers
            g.add("weights", "attention", comp["attention"] * frac / att)
            # a tensor-parallel group splits the attention heads only: every rank runs the whole FFN of the rows it
            # owns, so dense / shared / routed expert weights and the head are whole on each of its GPUs
            g.add("weights", "dense_ffn", comp["dense_ffn"] * frac)
            g.add("weights", "shared_experts", comp["shared_experts"] * frac)
            g.add("weights", "router+norms", (comp["router"] + comp["norms"]) * frac)
            g.add("weights", "indexer", comp["indexer"] * frac / att)
            if s == 0:
                g.add("weights", "embedding", comp["embedding"])
            if s == pp - 1:
                g.add("weights", "head", comp["head"])
                if spec == "mtp":
                    g.add("weights", "mtp", comp["mtp"] / att if colocated else
                          (comp["mtp"] - cfg.mtp_layers * cfg.num_experts * weight_bytes(cfg.expert_params(), req.expert_format or cfg.weight_format)) / att)
            if colocated and cfg.num_experts:
                lo, hi = (0, cfg.num_experts) if att > 1 else ranges[s * att + t]
                g.add("experts", f"experts[{lo}:{hi}]", comp["one_expert_all_layers"] * (hi - lo) * frac
                      + req.redundant_experts * comp["one_expert_all_layers"] * frac)
            width = cfg.hidden * 2
            qkv = (cfg.num_heads * cfg.qk_head_dim * 3 if cfg.is_mla else (cfg.num_heads + 2 * cfg.num_kv_heads) * cfg.head_dim) * 2
            g.add("workspace", "activations", act_rows * (4 * width + 2 * qkv // att + cfg.dense_ffn * 2 // att))
            g.add("workspace", "logits", req.decode_rows * cfg.vocab_size * 4)
            if cfg.num_experts:
                g.add("exchange", "combine+routes", act_rows * cfg.top_k * (cfg.hidden * 2 + 12))
                if colocated:
                    rows = act_rows * cfg.top_k + e_max * 128
                    g.add("exchange", "slab+fc1", rows * (cfg.hidden + cfg.expert_ffn) * 2)
            if req.graph_reserve_bytes is None:
                g.add("graphs", "decode graphs (default)", (256 << 20) * req.decode_lanes)
            else:
                g.add("graphs", f"decode graphs ({req.graph_reserve_source})", req.graph_reserve_bytes * req.decode_lanes)
            g.add("reserve", "context+slack", req.gpu_memory_cap * req.reserve_fraction)
    # ---- expert devices ------------------------------------------------------------------------------
    for r in range(exp):
        g = devices[att * pp + r]
        g.role = "expert"
        lo, hi = ranges[r]
        g.add("experts", f"experts[{lo}:{hi}]", comp["one_expert_all_layers"] * (hi - lo + req.redundant_experts))
        if spec == "mtp":
            g.add("experts", "mtp experts", cfg.mtp_layers * (hi - lo) * weight_bytes(cfg.expert_params(), req.expert_format or cfg.weight_format))
        rows = act_rows * cfg.top_k + e_max * 128
        g.add("exchange", "slab+fc1", rows * (cfg.hidden + cfg.expert_ffn) * 2 * req.decode_lanes)
        g.add("graphs", "expert graphs", 128 << 20)
        g.add("reserve", "context+slack", req.gpu_memory_cap * req.reserve_fraction)
    # ---- KV pool: what is left on the tightest attention device ----------------------------------------
    att_devs = devices[: att * pp]
    for g in devices[:n_dev]:
        if g.free < 0:
            worst = max(g.by_category().items(), key=lambda kv: kv[1])
            return Placement(False, f"GPU {g.index} ({g.role}) over capacity by {(-g.free)/GIB:.1f} GiB; largest demand {worst[0]} "
                             f"{worst[1]/GIB:.1f} GiB", "", att, exp, pp, devices, ranges, 0, kv_per_token_dev, 0, spec, req.decode_lanes)
    room = min(g.free for g in att_devs)
    pool_tokens = min(req.pool_tokens_target, room // max(kv_per_token_dev, 1))
    pool_tokens -= pool_tokens % 64
    pool_min = min(req.pool_tokens_min, req.pool_tokens_target)
    if pool_tokens < pool_min:
        return Placement(False, f"KV pool would hold {pool_tokens} tokens, minimum is {pool_min}", "", att, exp, pp, devices,
                         ranges, pool_tokens, kv_per_token_dev, 0, spec, req.decode_lanes)
    for g in att_devs:
        g.add("kv_pool", f"{pool_tokens} tokens", pool_tokens * kv_per_token_dev)
    conc = pool_tokens // max(req.max_context_tokens, 1)
    if conc < req.concurrency:
        notes.append(f"pool admits {conc} sequences at the full {req.max_context_tokens}-token context (requested concurrency {req.concurrency}); "
                     "longer sequences stall admission rather than truncate")
    layout = (f"attention tp{att}" + (f" x pp{pp}" if pp > 1 else "") + (f" + experts ep{exp}" if exp else " + experts colocated"))
    # ---- throughput proxy for "auto": decode step bytes on the busiest device ---------------------------
    act_exp = min(cfg.num_experts, req.concurrency * cfg.top_k) if cfg.num_experts else 0
    exp_dev = exp if exp else pp
    t_experts = comp["one_expert_all_layers"] * act_exp / max(exp_dev, 1)
    t_backbone = (comp["attention"] + comp["dense_ffn"] + comp["shared_experts"] + comp["head"]) / att \
        + req.concurrency * min(req.max_context_tokens, 8192) * kv_tok_layer * cfg.num_layers / kv_shard
    step = (t_experts + t_backbone) if colocated else max(t_experts, t_backbone) + 0.35 * min(t_experts, t_backbone)
    return Placement(True, "ok", layout, att, exp, pp, devices, ranges, pool_tokens, kv_per_token_dev, conc, spec,
                     req.decode_lanes, notes, score=1.0 / max(step, 1.0))


def kernel_geometry(cfg: ModelConfig) -> str:
    """Why the CUDA engines cannot run this geometry ("" = they can): their attention kernels are written for one head
    shape per family."""
    if cfg.is_mla:
        if (cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.qk_nope_dim, cfg.v_head_dim) != (512, 64, 128, 128):
            return "the MLA kernels take the DeepSeek shape (latent 512, rope 64, nope 128, value 128)"
        if 128 % cfg.num_heads:
            return "the MLA kernels take a head count that divides 128"
        return ""
    if cfg.head_dim != 128:
        return "the GQA kernels take head_dim 128"
    g = cfg.num_heads // max(cfg.num_kv_heads, 1)
    if cfg.num_heads % max(cfg.num_kv_heads, 1) or g > 16 or 16 % g:
        return "the GQA decode kernel takes 1, 2, 4, 8 or 16 query heads per kv head"
    return ""


def engine_for(cfg: ModelConfig, att: int, exp: int, pp: int) -> tuple[str, str]:
    """(engine that serves the layout, note).  The solver sizes any (attention TP, expert EP, stages) split; this names
    the code path that runs it, so a plan never silently proposes a layout nothing can execute."""
    why = kernel_geometry(cfg)
    if why:
        return "", why + "; the CPU oracle serves this checkpoint (serve --fake-engine)"
    if pp > 1:
        if att == 1 and exp == 0 and not cfg.is_mla:
            return "pp", "layer ranges as pipeline stages with ring hops (models/pp_gqa.py)"
        return "", "pipeline stages are wired for the GQA family alone (no tensor parallelism or expert ranks beside them)"
    if att == 1:
        return ("afd", "attention on one GPU, routed experts on the others (parallel/afd.py)") if exp else \
               ("single", "attention and experts on one GPU")
    if exp == 0 and not cfg.is_mla and cfg.num_kv_heads % att == 0:
        return "tp", "heads split over the GPUs, residual rows sharded, experts replicated (models/tp_gqa.py)"
    if exp == 0 and cfg.is_mla and not cfg.indexer_heads and cfg.num_heads % att == 0 and 128 % (cfg.num_heads // att) == 0:
        return "tp", "MLA heads split over the GPUs, latent cache replicated, residual rows sharded (models/tp_mla.py)"
    if exp == 0:
        return "", ("tensor-parallel attention needs kv heads (GQA) or heads (dense MLA, at most 128 per rank) divisible by the degree; "
                    "the lightning indexer is not split")
    return "", ("a tensor-parallel attention group in front of the expert exchange is not wired; the benchmark's 2 + 6 and 4 + 4 layouts "
                "run data-parallel attention replicas instead (bench.py --attention-ranks), which the HTTP server does not drive")


# What ``serve`` / ``launch`` can start: one attention rank with or without expert ranks, or a tensor-parallel attention
# group whose rank 0 holds the scheduler and whose other ranks repeat its steps (parallel/mirror.py)
HTTP_ENGINES = ("single", "afd", "tp")


def candidates(req: PlacementRequest) -> list[tuple[int, int, int]]:
    cfg = req.cfg
    out = []
    att_opts = [req.attention_ranks] if req.attention_ranks else [a for a in (1, 2, 4, 8) if a <= req.gpus and cfg.num_heads % a == 0]
    for a in att_opts:
        pp = req.pipeline_stages
        rest = req.gpus - a * pp
        if req.expert_ranks is not None:
            exp_opts = [req.expert_ranks]
        elif not cfg.num_experts:
            exp_opts = [0]
        else:
            exp_opts = sorted({0} | ({rest} if rest > 0 else set())) if rest >= 0 else []      # colocated, or every other GPU
        for e in exp_opts:
            if e >= 0 and a * pp + e <= req.gpus:
                out.append((a, e, pp))
    return out


def solve(req: PlacementRequest) -> Placement:
    """Best feasible placement, or the most informative failure."""
    best: Placement | None = None
    fail: Placement | None = None
    for a, e, pp in candidates(req):
        p = _place(req, a, e, pp)
        p.engine, why = engine_for(req.cfg, a, e, pp)
        p.notes.append(("served by: " if p.engine else "not served yet: ") + why)
        # a layout an engine runs today wins over a faster-looking one that nothing executes
        if p.ok and (best is None or (bool(p.engine), p.score) > (bool(best.engine), best.score)):
            best = p
        elif not p.ok and fail is None:
            fail = p
    if best is not None:
        return best
    if fail is not None:
        return fail
    return Placement(False, "no candidate layout for this inventory", "", 0, 0, 1, [], [], 0, 0, 0, "off", 1)


def solve_frozen(req: PlacementRequest, attention_ranks: int, expert_ranks: int, pipeline_stages: int = 1) -> Placement:
    """Re-check a layout decided earlier (runtime admission against the planned baseline)."""
    p = _place(req, attention_ranks, expert_ranks, pipeline_stages)
    p.engine, why = engine_for(req.cfg, attention_ranks, expert_ranks, pipeline_stages)
    p.notes.append(("served by: " if p.engine else "not served yet: ") + why)
    return p
