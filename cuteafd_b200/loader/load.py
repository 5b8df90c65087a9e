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
    view: "object | None" = None              # loader.mc.Selected for a multi-core repository

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


def open_snapshot(path: str, core_view: str | None = None) -> OpenedSnapshot:
    """``core_view``: which dense-core variant of a multi-core repository to open (None: ``$CUTEAFD_CORE_VIEW``, default
    ``original``); a plain checkpoint accepts ``original`` only."""
    from .snapshot import core_view as select_view, view_weight_map
    path = resolve(path)
    sel = select_view(path, core_view)
    cfg, hf = read_config(path, core_view)
    cat = Catalog(path, rename=families.canonical_name, weight_map=view_weight_map(path, core_view))
    ops = formats.detect_operands(cat)
    fam = families.detect(hf)
    model = fam.open(cfg, hf) if fam else None
    return OpenedSnapshot(path, cfg, hf, cat, ops, fam, model, sel)


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


STORED_EXPERT_FORMATS = {"fp8_block128": "fp8", "mxfp4": "mxfp4", "nvfp4": "nvfp4"}


def expert_storage_format(snap: OpenedSnapshot) -> str:
    """How the routed experts of a snapshot are served: "fp8" (E4M3 + 128x128 scales), "mxfp4", "nvfp4" keep the stored
    bytes; everything else (bf16 / f16 / f32, EXL3 trellis) is decoded to bf16 on load."""
    for pre, op in snap.operands.items():
        if ".mlp.experts." in pre:
            return STORED_EXPERT_FORMATS.get(op.format, "bf16")
    return "bf16"


def load_experts_as_stored(snap: OpenedSnapshot, lo: int, hi: int, device: torch.device) -> tuple[str, list[tuple]]:
    """Routed experts [lo, hi) of every MoE layer in the form the grouped GEMMs read, with the checkpoint's bytes
    untouched: no dequantisation and no re-encoding, only the per-expert tensors stacked along a new first dimension
    (what the reference calls slicing the stored tensors per rank: rust/crates/cuteafd-loader/src/formats/
    fp8_experts.rs:8-33,80-86).  Returns (format, [(gate, up, down) per MoE layer]) where each of the three is

      bf16    tensor [n, N, K]
      fp8     (E4M3 [n, N, K], fp32 block scales [n, N/128, K/128])           scales multiply, whatever their name
      mxfp4   (packed uint8 [n, N, K/2], UE8M0 uint8 [n, N, K/32], None)
      nvfp4   (packed uint8 [n, N, K/2], E4M3 scales as bytes [n, N, K/16], fp32 global multipliers [n])
    """
    cfg, cat, ops = snap.cfg, snap.catalog, snap.operands
    fmt = expert_storage_format(snap)
    out = []
    for i in range(cfg.num_layers + cfg.mtp_layers):
        if not (cfg.is_moe_layer(i) if i < cfg.num_layers else cfg.num_experts > 0):
            continue
        trio = []
        for proj in ("gate_proj", "up_proj", "down_proj"):
            names = [f"model.layers.{i}.mlp.experts.{e}.{proj}" for e in range(lo, hi)]
            if names[0] not in ops:
                trio = []
                break
            for nme in names:
                got = STORED_EXPERT_FORMATS.get(ops[nme].format, "bf16")
                if got != fmt:
                    raise ValueError(f"{nme}: stored as {ops[nme].format}, the layer's other experts as {fmt}")
            if fmt == "bf16":
                trio.append(torch.stack([formats.dequantize(ops[nme], cat).to(torch.bfloat16) for nme in names]).to(device).contiguous())
                continue
            # stacked as raw bytes (one copy per tensor, no arithmetic), then viewed back in the stored dtype
            first = cat.read(ops[names[0]].weight)
            payload = torch.stack([cat.read(ops[nme].weight).view(torch.uint8) for nme in names]).to(device).contiguous()
            scales = torch.stack([cat.read(ops[nme].scale_tensor) for nme in names])
            if fmt == "fp8":
                payload = payload.view(first.dtype)
                if ops[names[0]].block_scale is None or ops[names[0]].block_scale.rows != 128 or ops[names[0]].block_scale.cols != 128:
                    raise ValueError(f"{names[0]}: E4M3 experts need 128x128 block scales")
                trio.append((payload, scales.float().to(device).contiguous()))
            elif fmt == "mxfp4":
                trio.append((payload, scales.view(torch.uint8).to(device).contiguous(), None))
            else:
                glob = torch.cat([cat.read(ops[nme].global_scale).float().reshape(1) if ops[nme].global_scale else torch.ones(1)
                                  for nme in names])
                trio.append((payload, scales.view(torch.uint8).to(device).contiguous(), glob.to(device).contiguous()))
        if trio:
            out.append(tuple(trio))
    return fmt, out


def attach_stored_experts(W, snap: OpenedSnapshot, device: torch.device) -> str:
    """Give an engine weight set (built without experts) its routed experts in their stored form.  Sets
    ``W.expert_format`` and each MoE layer's ``w_gate / w_up / w_down``."""
    cfg = snap.cfg
    fmt, stacks = load_experts_as_stored(snap, 0, cfg.num_experts, device)
    it = iter(stacks)
    for i, L in enumerate(W.layers):
        if L.router is not None:
            L.w_gate, L.w_up, L.w_down = next(it)
    W.expert_format = fmt
    return fmt


FP8_TWIN_PROJECTIONS = {"wq_b": "self_attn.q_b_proj", "wo": "self_attn.o_proj", "s_gate": "mlp.shared_experts.gate_proj",
                        "s_up": "mlp.shared_experts.up_proj", "s_down": "mlp.shared_experts.down_proj"}


def attach_fp8_twins(W, snap: "OpenedSnapshot | None" = None, device: torch.device | None = None, only: set[str] | None = None) -> int:
    """E4M3 twins (values + 128x128 block scales) of the large backbone projections for decode-sized steps: q_b, the
    o projection and the shared expert.  From a snapshot that stores them as E4M3-block128 the twins are the stored
    bytes, untouched; otherwise (bf16 checkpoint, random init) they are encoded once from the bf16 weights.  Returns the
    number of projections that got a twin."""
    from ..quant import codecs
    n = 0
    for i, L in enumerate(W.layers):
        twins = {}
        for attr, tensor in FP8_TWIN_PROJECTIONS.items():
            w = getattr(L, attr, None)
            if w is None or not torch.is_tensor(w) or w.shape[0] % 128 or w.shape[1] % 128:
                continue
            if only is not None and f"model.layers.{i}.{tensor}.weight" not in only:
                continue                                  # the fp8-compact view converts its declared core, nothing else
            op = snap.operands.get(f"model.layers.{i}.{tensor}") if snap is not None else None
            if op is not None and op.format == "fp8_block128" and op.block_scale is not None and (op.block_scale.rows, op.block_scale.cols) == (128, 128):
                q = snap.catalog.read(op.weight).to(device or w.device).contiguous()
                sc = snap.catalog.read(op.scale_tensor).float().to(device or w.device).contiguous()
            else:
                q, sc = codecs.fp8_quant_block128(w.float())
                q, sc = q.contiguous(), sc.float().contiguous()
            twins[attr] = (q, sc)
            n += 1
        L.fp8 = twins or None
    return n


def random_stored_experts(W, cfg, fmt: str, device: torch.device, seed: int = 0, std: float = 0.02) -> str:
    """Random routed experts in a stored format ("fp8", "mxfp4", "nvfp4"), generated and encoded on the device one
    expert at a time, attached to ``W`` the way ``attach_stored_experts`` attaches a checkpoint's (benchmarks of the
    quantised serving paths without a checkpoint on disk).  MTP layers' experts included."""
    from ..quant import codecs
    g = torch.Generator(device=device).manual_seed(seed)
    E, I, H = cfg.num_experts, cfg.expert_ffn, cfg.hidden

    def stack(rows: int, cols: int):
        parts = []
        for _ in range(E):
            w = torch.empty(rows, cols, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
            if fmt == "fp8":
                parts.append(codecs.fp8_quant_block128(w))
            elif fmt == "mxfp4":
                parts.append(codecs.mxfp4_quant(w))
            else:
                q, bs, glob = codecs.nvfp4_quant(w)
                parts.append((q, bs.view(torch.uint8), glob))
        cols_ = list(zip(*parts))
        if fmt == "fp8":
            return torch.stack(cols_[0]).contiguous(), torch.stack(cols_[1]).float().contiguous()
        if fmt == "mxfp4":
            return torch.stack(cols_[0]).contiguous(), torch.stack(cols_[1]).contiguous(), None
        return torch.stack(cols_[0]).contiguous(), torch.stack(cols_[1]).contiguous(), torch.cat(cols_[2]).contiguous()
    assert fmt in ("fp8", "mxfp4", "nvfp4"), fmt
    for L in W.layers:
        if L.router is not None:
            L.w_gate, L.w_up, L.w_down = stack(I, H), stack(I, H), stack(H, I)
    W.expert_format = fmt
    return fmt


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


def host_embedding_table(path: str, **kw):
    """The snapshot's token embedding as a memory-mapped host table (``--embedding-placement host``): rows are gathered
    per step instead of the table living in GPU memory.  bf16 / f16 / f32 tables only (a quantised embedding is
    refused by the family's format rules anyway)."""
    from .mapped_table import MappedTable
    snap = open_snapshot(path)
    name = "model.embed_tokens.weight"
    if name not in snap.catalog.entries:
        raise ValueError(f"{path}: no {name} to map")
    if snap.catalog.entries[name].dtype != "BF16":
        raise ValueError("a host-resident embedding table is read as stored: it must be bf16 in the checkpoint")
    return MappedTable.from_safetensors(snap.catalog, name, **kw)


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
    stored = expert_storage_format(snap) if cfg.num_experts else "bf16"
    if cfg.is_mla:
        from ..models.mla_moe import LatentCache, MlaMoeEngine, MlaMoeWeights
        if stored != "bf16":             # quantised experts stay as stored; the rest of the model is decoded to bf16
            _, params = load_params(path, dtype=torch.bfloat16, exclude=".mlp.experts.")
            W = MlaMoeWeights.from_params(cfg, params, device, with_experts=False)
            attach_stored_experts(W, snap, device)
        else:
            _, params = load_params(path, dtype=torch.bfloat16)
            W = MlaMoeWeights.from_params(cfg, params, device)
        if cfg.weight_format == "fp8_block128":
            attach_fp8_twins(W, snap, device)
        elif snap.view is not None and snap.view.convert_fp8:
            attach_fp8_twins(W, None, device, only=set(snap.view.view.core_tensors))      # encoded once, here, from bf16
        return cfg, MlaMoeEngine(cfg, W, LatentCache(cfg, num_pages, device), max_tokens=max_tokens, max_seqs=max_seqs)
    from ..models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
    if snap.view is not None and snap.view.convert_fp8:
        raise ValueError("core view fp8-compact: only the MLA engine runs E4M3 backbone projections; serve this "
                         "checkpoint with the original or a stored compact view")
    if stored != "bf16":
        _, params = load_params(path, dtype=torch.bfloat16, exclude=".mlp.experts.")
        W = GqaMoeWeights.from_params(cfg, params, device, with_experts=False)
        attach_stored_experts(W, snap, device)
    elif cfg.mtp_layers or cfg.attention_bias:
        _, params = load_params(path, dtype=torch.bfloat16)
        W = GqaMoeWeights.from_params(cfg, params, device)
    else:
        _, W = load_gqa_engine_weights(path, device)
    return cfg, GqaMoeEngine(cfg, W, KvCache(cfg, num_pages, device), max_tokens=max_tokens, max_seqs=max_seqs)
