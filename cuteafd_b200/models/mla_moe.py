"""MLA + MoE decoder (DeepSeek-V3 geometry: kv_lora 512, rope 64, nope 128, v 128) on the sm_100a kernels.

Attention runs in the absorbed form for every step shape: the cache holds one [512 latent | 64 rope]
record per token (shared by all heads), queries are moved into latent space per head
(q_nope @ W_uk), one tcgen05 kernel attends over the paged latent cache, and the latent output is
moved back per head (@ W_uv) before o_proj.  The two per-head projections run as *grouped* GEMMs
with the heads in the role of experts, so a layer's attention is nine launches at any token count:

    fused q_a/kv_a GEMM -> norm + rope + cache write -> q_b GEMM -> q split/rope -> absorb (grouped)
    -> MLA attention (+ merge when split) -> un-absorb (grouped) -> o_proj (+ residual)

The FFN half (dense SwiGLU / routed experts with shared expert) is shared with the GQA engine.
Reference counterparts: the GLM-5 / DeepSeek attention unit programs
(rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2110-2262), absorbed and sparse MLA
kernels (native/shared/cuda/attention.cu:249-925), compose kernels (native/shared/cuda/mla_indexing.cu:46).
"""
from __future__ import annotations

import math

import torch

from ..config import ModelConfig
from ..ops import kernels as K
from ..parallel.moe_exchange import ExchangeGeometry, LocalExchange
from .gqa_moe import PAGE, Batch, GqaMoeEngine, LayerWeights, MtpExtras, layer_is_moe, load_mtp_extras

REC = 576


class MlaLayerWeights(LayerWeights):
    __slots__ = ("wqkv_a", "q_a_norm", "kv_a_norm", "wq_b", "w_uk", "w_uv", "wq_idx", "w_kb")

    def __init__(self) -> None:
        for s in LayerWeights.__slots__ + MlaLayerWeights.__slots__:
            setattr(self, s, None)


class MlaMoeWeights:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self.embed = self.final_norm = self.lm_head = None
        self.layers: list[MlaLayerWeights] = []
        self.mtp: list[MtpExtras] = []

    @staticmethod
    def _split_kv_b(cfg: ModelConfig, kv_b: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """kv_b_proj [heads * (nope + v), kv_lora] -> W_uk [heads, kv_lora, nope] (absorb weight, out = latent)
        and W_uv [heads, v, kv_lora]."""
        w = kv_b.view(cfg.num_heads, cfg.qk_nope_dim + cfg.v_head_dim, cfg.kv_lora_rank)
        return w[:, :cfg.qk_nope_dim].transpose(1, 2).contiguous(), w[:, cfg.qk_nope_dim:].contiguous()

    @staticmethod
    def from_params(cfg: ModelConfig, p: dict[str, torch.Tensor], device: torch.device,
                    with_experts: bool = True) -> "MlaMoeWeights":
        def t(name: str) -> torch.Tensor:
            return p[name].to(device=device, dtype=torch.bfloat16).contiguous()

        W = MlaMoeWeights(cfg)
        W.embed, W.final_norm = t("model.embed_tokens.weight"), t("model.norm.weight")
        W.lm_head = W.embed if cfg.tie_embeddings else t("lm_head.weight")
        W.mtp = load_mtp_extras(cfg, p, t)
        for i in range(cfg.num_layers + cfg.mtp_layers):
            pre, L = f"model.layers.{i}.", MlaLayerWeights()
            a, m = pre + "self_attn.", pre + "mlp."
            L.ln1, L.ln2 = t(pre + "input_layernorm.weight"), t(pre + "post_attention_layernorm.weight")
            if cfg.q_lora_rank:
                L.wqkv_a = torch.cat([t(a + "q_a_proj.weight"), t(a + "kv_a_proj_with_mqa.weight")]).contiguous()
                L.q_a_norm, L.wq_b = t(a + "q_a_layernorm.weight"), t(a + "q_b_proj.weight")
            else:
                L.wqkv_a, L.wq_b = t(a + "kv_a_proj_with_mqa.weight"), t(a + "q_proj.weight")
            L.kv_a_norm = t(a + "kv_a_layernorm.weight")
            if cfg.indexer_heads:      # index keys and head weights ride on the fused q_a / kv_a projection
                L.wqkv_a = torch.cat([L.wqkv_a, t(a + "indexer.wk.weight"), t(a + "indexer.weights_proj.weight")]).contiguous()
                L.wq_idx = t(a + "indexer.wq.weight")
            L.w_uk, L.w_uv = MlaMoeWeights._split_kv_b(cfg, t(a + "kv_b_proj.weight"))
            L.w_kb = L.w_uk.transpose(1, 2).reshape(cfg.num_heads * cfg.qk_nope_dim, cfg.kv_lora_rank).contiguous()
            L.wo = t(a + "o_proj.weight")
            if layer_is_moe(cfg, i):
                L.router = t(m + "gate.weight")
                b = p.get(m + "gate.e_score_correction_bias")
                L.router_bias = None if b is None else b.to(device=device, dtype=torch.float32).contiguous()
                for dst, src in ((("w_gate", "gate_proj"), ("w_up", "up_proj"), ("w_down", "down_proj")) if with_experts else ()):
                    setattr(L, dst, torch.stack([t(m + f"experts.{e}.{src}.weight") for e in range(cfg.num_experts)]).contiguous())
                if cfg.num_shared_experts:
                    L.s_gate, L.s_up, L.s_down = (t(m + f"shared_experts.{n}_proj.weight") for n in ("gate", "up", "down"))
            else:
                L.d_gate, L.d_up, L.d_down = (t(m + f"{n}_proj.weight") for n in ("gate", "up", "down"))
            W.layers.append(L)
        return W

    @staticmethod
    def random_init(cfg: ModelConfig, device: torch.device, seed: int = 0, std: float = 0.02,
                    with_experts: bool = True) -> "MlaMoeWeights":
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape: int) -> torch.Tensor:
            out = torch.empty(*shape, dtype=torch.bfloat16, device=device)
            out.normal_(0.0, std, generator=g)
            return out

        def ones(n: int) -> torch.Tensor:
            return torch.ones(n, dtype=torch.bfloat16, device=device)

        H = cfg.hidden
        W = MlaMoeWeights(cfg)
        W.embed, W.final_norm = w(cfg.vocab_size, H), ones(H)
        W.lm_head = W.embed if cfg.tie_embeddings else w(cfg.vocab_size, H)
        W.mtp = [MtpExtras(ones(H), ones(H), w(H, H), w(H, H), ones(H)) for _ in range(cfg.mtp_layers)]
        for i in range(cfg.num_layers + cfg.mtp_layers):
            L = MlaLayerWeights()
            L.ln1, L.ln2 = ones(H), ones(H)
            L.wqkv_a = w(cfg.q_lora_rank + REC + ((cfg.indexer_dim + cfg.indexer_heads) if cfg.indexer_heads else 0), H)
            L.wq_idx = w(cfg.indexer_heads * cfg.indexer_dim, H) if cfg.indexer_heads else None
            L.q_a_norm = ones(cfg.q_lora_rank) if cfg.q_lora_rank else None
            L.kv_a_norm = ones(cfg.kv_lora_rank)
            L.wq_b = w(cfg.num_heads * cfg.qk_head_dim, cfg.q_lora_rank or H)
            L.w_uk, L.w_uv = w(cfg.num_heads, cfg.kv_lora_rank, cfg.qk_nope_dim), w(cfg.num_heads, cfg.v_head_dim, cfg.kv_lora_rank)
            L.w_kb = L.w_uk.transpose(1, 2).reshape(cfg.num_heads * cfg.qk_nope_dim, cfg.kv_lora_rank).contiguous()
            L.wo = w(H, cfg.num_heads * cfg.v_head_dim)
            if layer_is_moe(cfg, i):
                L.router = w(cfg.num_experts, H)
                L.router_bias = torch.zeros(cfg.num_experts, dtype=torch.float32, device=device) if cfg.router_bias else None
                if with_experts:
                    L.w_gate, L.w_up = w(cfg.num_experts, cfg.expert_ffn, H), w(cfg.num_experts, cfg.expert_ffn, H)
                    L.w_down = w(cfg.num_experts, H, cfg.expert_ffn)
                if cfg.num_shared_experts:
                    inter = cfg.expert_ffn * cfg.num_shared_experts
                    L.s_gate, L.s_up, L.s_down = w(inter, H), w(inter, H), w(H, inter)
            else:
                L.d_gate, L.d_up, L.d_down = w(cfg.dense_ffn, H), w(cfg.dense_ffn, H), w(H, cfg.dense_ffn)
            W.layers.append(L)
        return W


class LatentCache:
    """Paged latent pools, one per layer.  bf16 records: [num_pages, 64, 576] (1152 bytes per token and layer, for all
    heads).  FP8 records (``cfg.kv_format == "fp8_ds_mla"``): [num_pages, 64, 656] bytes = 512 E4M3 latents, 4 fp32
    scales, 64 bf16 rope dims; served by the sparse-attention path only.  Page 0 stays all-zero."""

    def __init__(self, cfg: ModelConfig, num_pages: int, device: torch.device):
        self.num_pages = num_pages
        n = cfg.num_layers + cfg.mtp_layers
        self.fp8 = cfg.kv_format == "fp8_ds_mla"
        if self.fp8:
            assert cfg.indexer_heads, "FP8 latent records are read by the sparse (indexer) attention path"
            self.c = [torch.zeros(num_pages, PAGE, K.FP8_RECORD_BYTES, dtype=torch.uint8, device=device) for _ in range(n)]
        else:
            self.c = [torch.zeros(num_pages, PAGE, REC, dtype=torch.bfloat16, device=device) for _ in range(n)]
        # index keys of the lightning indexer, paged like the latent records
        self.idx = ([torch.zeros(num_pages, PAGE, cfg.indexer_dim, dtype=torch.bfloat16, device=device) for _ in range(n)]
                    if cfg.indexer_heads else [])

    def bytes_per_page(self) -> int:
        return sum(t[0].numel() * t.element_size() for t in self.c + self.idx)

    def copy_page(self, src: int, dst: int) -> None:
        for c in self.c + self.idx:
            c[dst].copy_(c[src])


class _HeadTiles:
    """Tile table that lets the grouped GEMM treat heads as experts over a head-major slab [heads, t_pad, *]."""

    def __init__(self, T: int, heads: int, device: torch.device):
        self.tile_rows = 16 if T <= 16 else 32 if T <= 32 else 64 if T <= 64 else 128
        per_head = (T + self.tile_rows - 1) // self.tile_rows
        self.t_pad = per_head * self.tile_rows
        i32 = dict(dtype=torch.int32, device=device)
        h = torch.arange(heads, **i32)
        self.tile_expert = h.repeat_interleave(per_head).contiguous()
        self.tile_row0 = (h[:, None] * self.t_pad + torch.arange(per_head, **i32)[None, :] * self.tile_rows).reshape(-1).contiguous()
        self.max_tiles = heads * per_head
        self.num_tiles = torch.tensor([self.max_tiles], **i32)
        t = torch.arange(self.t_pad, **i32)
        dst = t[None, :] * heads + h[:, None]
        self.row_dst = torch.where(t[None, :] < T, dst, torch.full_like(dst, -1)).reshape(-1).contiguous()


class MlaMoeEngine(GqaMoeEngine):
    """Single-GPU MLA engine; shares the FFN half, the logits head and greedy selection with the GQA engine."""
    EXPANDED_PREFILL_TOKENS = 64     # fresh prompt chunks of at least this many tokens use the expanded-form attention
    GATHER_BLOCKS = 128              # query tokens per FP8 gather + attention pass (2048 records each: 302 MB of bf16)

    def __init__(self, cfg: ModelConfig, weights: MlaMoeWeights, kv: LatentCache, max_tokens: int, max_seqs: int = 64,
                 build_moe: bool = True):
        assert cfg.is_mla and cfg.kv_lora_rank == 512 and cfg.qk_rope_dim == 64 and cfg.qk_nope_dim == 128 and cfg.v_head_dim == 128
        assert 128 % cfg.num_heads == 0, "local head count must divide 128"
        assert not cfg.indexer_heads or (cfg.indexer_dim == 128 and cfg.indexer_heads in (32, 64, 128, 256))
        self.cfg, self.W, self.kv = cfg, weights, kv
        self.device = dev = weights.embed.device
        self.max_tokens = max_tokens
        H, heads = cfg.hidden, cfg.num_heads
        bf = dict(dtype=torch.bfloat16, device=dev)

        class _Ws:
            pass
        ws = self.ws = _Ws()
        ws.h, ws.x = torch.empty(max_tokens, H, **bf), torch.empty(max_tokens, H, **bf)
        ws.a = torch.empty(max_tokens, cfg.q_lora_rank + REC + ((cfg.indexer_dim + cfg.indexer_heads) if cfg.indexer_heads else 0), **bf)
        ws.q_idx = torch.empty(max_tokens, cfg.indexer_heads * cfg.indexer_dim, **bf) if cfg.indexer_heads else None
        ws.sel = torch.empty(max_tokens, cfg.indexer_topk, dtype=torch.int32, device=dev) if cfg.indexer_heads else None
        ws.scores = None
        ws.q_a = torch.empty(max_tokens, cfg.q_lora_rank, **bf) if cfg.q_lora_rank else None
        ws.q = torch.empty(max_tokens, heads * cfg.qk_head_dim, **bf)
        t_pad_max = ((max_tokens + 127) // 128) * 128
        ws.q_slab = torch.zeros(heads * t_pad_max * 128, **bf)
        ws.q_abs = torch.empty(max_tokens, heads, REC, **bf)
        ws.o_slab = torch.zeros(heads * t_pad_max * 512, **bf)
        ws.attn = torch.empty(max_tokens, heads * cfg.v_head_dim, **bf)
        ws.router = torch.empty(max_tokens, max(cfg.num_experts, 1), dtype=torch.float32, device=dev)
        dense = cfg.first_dense_layers > 0 or cfg.num_experts == 0
        ws.ffn_d = torch.empty(max_tokens, cfg.dense_ffn, **bf) if dense else None
        ws.ffn_s = torch.empty(max_tokens, cfg.expert_ffn * cfg.num_shared_experts, **bf) if cfg.num_shared_experts else None
        ws.shared = torch.empty(max_tokens, H, **bf) if cfg.num_shared_experts else None
        from ..ref.ops import rope_inv_freq, rope_magnitudes
        mag, scale_mul = rope_magnitudes(cfg)
        if mag != 1.0:
            raise ValueError("a YaRN configuration whose cos / sin magnitude differs from 1 (mscale != mscale_all_dim) is not supported")
        self.inv_freq = rope_inv_freq(cfg, cfg.qk_rope_dim).to(dev)           # YaRN / linear scaling is in this table
        self.scale = scale_mul / math.sqrt(cfg.qk_head_dim)                    # DeepSeek YaRN: mscale(all_dim)^2 on the logits
        self.moe = None
        self.pre_moe = None
        if cfg.num_experts and build_moe:
            self.moe = LocalExchange(ExchangeGeometry(H, cfg.expert_ffn, cfg.num_experts, cfg.top_k, max_tokens, 1), dev)
        self.route_kw = dict(scoring=cfg.scoring, num_groups=cfg.num_groups, topk_groups=cfg.topk_groups,
                             normalize=cfg.norm_topk_prob, routed_scale=cfg.routed_scale)
        self.logits = torch.empty(min(max_seqs, max_tokens), cfg.vocab_size, dtype=torch.float32, device=dev)
        self.next_tokens = torch.empty(self.logits.shape[0], dtype=torch.int32, device=dev)
        self._scratch: torch.Tensor | None = None
        self.fixed_kv_split = K.batch_invariant_from_env()     # tokens per kv split in the batch-invariant form, else 0
        self.kv_exchange = None                                # context split: parallel.context_split.DeviceContextSplit
        self._tiles: dict[int, _HeadTiles] = {}
        self.select_hook = None      # callable(layer, selection [T, top_k]) for tests and traces (eager mode only)
        self._zero1 = torch.zeros(1, dtype=torch.int32, device=dev)
        self._blocks: dict[tuple[int, int, int], tuple[torch.Tensor, torch.Tensor]] = {}
        self.launches = 0
        self._f8_rows = {}

    def _block_table(self, S: int, max_q_len: int, per: int | None = None) -> tuple[torch.Tensor, torch.Tensor]:
        """Row blocks of the attention / indexer kernels: every sequence gets ceil(max_q_len / tokens per block)
        blocks; a block past a shorter sequence's new tokens does nothing."""
        per = per or 128 // self.cfg.num_heads
        key = (S, max_q_len, per)
        if key not in self._blocks:
            nb = (max_q_len + per - 1) // per
            i32 = dict(dtype=torch.int32, device=self.device)
            seq = torch.arange(S, **i32).repeat_interleave(nb).contiguous()
            tok0 = (torch.arange(nb, **i32) * per).repeat(S).contiguous()
            self._blocks[key] = (seq, tok0)
        return self._blocks[key]

    def _attention(self, i: int, T: int, b: Batch) -> None:
        cfg, L, ws = self.cfg, self.W.layers[i], self.ws
        heads, ql = cfg.num_heads, cfg.q_lora_rank
        if T not in self._tiles:
            self._tiles[T] = _HeadTiles(T, heads, self.device)
        ht = self._tiles[T]
        # A fresh prompt chunk (one sequence from position 0) of some length attends in the expanded form: kv_b applied
        # to the chunk's latents gives per-head K_nope / V, the scores take 128 + 64 dims and the values 128, a third of
        # the absorbed form's work (576 / 512).  Decode, continued chunks and sparse attention stay absorbed.
        expanded = b.prefill and b.fresh and not cfg.indexer_heads and T >= self.EXPANDED_PREFILL_TOKENS
        if expanded and getattr(ws, "lat", None) is None:
            bf = dict(dtype=torch.bfloat16, device=self.device)
            rows = ((self.max_tokens + 63) // 64) * 64
            ws.lat = torch.zeros(self.max_tokens, cfg.kv_lora_rank, **bf)
            ws.k_exp, ws.v_exp = torch.zeros(rows, heads * 128, **bf), torch.zeros(rows, heads * 128, **bf)
        self._proj_a(L, T)
        K.mla_prep_a(ws.a[:T, :ql + REC], ql, L.q_a_norm, L.kv_a_norm, self.inv_freq, b.positions, b.slots,
                     ws.q_a[:T] if ql else None, self.kv.c[i], cfg.rms_eps, cfg.rope_interleaved,
                     lat_out=ws.lat[:T] if expanded else None)
        self._linear(L, "wq_b", ws.q_a[:T] if ql else self._x_rows(T), ws.q[:T])
        q_slab = ws.q_slab[:heads * ht.t_pad * 128].view(heads, ht.t_pad, 128)
        o_slab = ws.o_slab[:heads * ht.t_pad * 512].view(heads, ht.t_pad, 512)
        # (the batch-invariant form keeps one absorb / un-absorb route for every decode width: the grouped GEMMs)
        small = T <= K.MLA_SMALL_ROWS and not expanded and not self.fixed_kv_split
        if small:
            # decode-sized step: nope / rope split, RoPE and the absorb projection in one launch
            K.mla_absorb_small(ws.q[:T], L.w_uk, self.inv_freq, b.positions, ws.q_abs[:T], heads, cfg.rope_interleaved)
        else:
            K.mla_q_split(ws.q[:T], self.inv_freq, b.positions, q_slab, ws.q_abs[:T], heads, cfg.rope_interleaved)
        if expanded:
            rows = ((T + 63) // 64) * 64
            K.linear(ws.lat[:T], L.w_kb, out=ws.k_exp[:T])
            K.linear(ws.lat[:T], L.w_uv.view(heads * 128, cfg.kv_lora_rank), out=ws.v_exp[:T])
            K.attn_prefill_mla(ws.q[:T], ws.q_abs[:T], ws.k_exp[:rows], ws.v_exp[:rows], self._zero1, self.kv.c[i], b.page_table,
                               b.seq_lens, b.q_start, ws.attn[:T], b.max_q_len, heads, self.scale)
            self._proj_o(L, T, twin=False)
            self.launches += 8
            return
        if not small:
            K.grouped_linear(q_slab.view(-1, 128), L.w_uk, ws.q_abs, ht.tile_expert, ht.tile_row0, ht.num_tiles, ht.max_tiles,
                             ht.tile_rows, row_dst=ht.row_dst, ldo=REC, split_k=False)
        S, max_pages = b.page_table.shape
        sel = self._select(i, T, b) if cfg.indexer_heads else None
        bseq, btok = self._block_table(S, b.max_q_len, 1 if sel is not None else None)
        nb = bseq.numel()
        if self.kv_exchange is not None:
            # context split: this rank holds a share of every sequence's records; partials meet in every rank's scratch
            self.kv_exchange.attend_mla(ws.q_abs[:T], self.kv.c[i], b.page_table, b.seq_lens, b.kv_base, b.q_start, bseq, btok,
                                        o_slab, self.scale, ht.t_pad)
            self._unabsorb(L, T, small, o_slab, ht)
            self.launches += (7 if small else 8) + 2 + self.kv_exchange.ranks
            return
        tiles = (min(cfg.indexer_topk, max_pages * 64) // 32) if sel is not None else max_pages * 2
        splits = 1 if b.prefill else max(1, min(K.num_sms() // max(1, nb * 2), max(1, tiles // 8), 32))
        if self.fixed_kv_split and not b.prefill:       # batch-invariant form: the split grid is a function of the table width only
            splits = K.kv_splits_fixed((tiles + 1) // 2, cap=64)
        if splits > 1:
            need = K.mla_scratch_floats(nb, splits)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
        if self.kv.fp8:
            # FP8 records: the selected records of a slice of query tokens are expanded to bf16 (the buffer stays in L2
            # for decode-sized steps) and the sparse kernel reads them from there
            k = sel.shape[1]
            per = min(nb, self.GATHER_BLOCKS)
            if getattr(ws, "gathered", None) is None or ws.gathered.numel() < max(per * k, 64) * REC:
                ws.gathered = torch.zeros(max(per * k, 64) * REC, dtype=torch.bfloat16, device=self.device)
            for b0 in range(0, nb, per):
                bs, bt = bseq[b0:b0 + per], btok[b0:b0 + per]
                K.mla_fp8_gather(self.kv.c[i], sel, b.page_table, b.seq_lens, b.q_start, bs, bt, ws.gathered)
                K.mla_attention(ws.q_abs[:T], None, b.page_table, b.seq_lens, b.q_start, bs, bt, o_slab, self.scale, splits,
                                self._scratch if splits > 1 else None, out_tpad=ht.t_pad, sparse_idx=sel, gathered=ws.gathered)
                self.launches += 1 + (1 if splits > 1 else 0) + (1 if b0 else 0)
        else:
            K.mla_attention(ws.q_abs[:T], self.kv.c[i], b.page_table, b.seq_lens, b.q_start, bseq, btok, o_slab, self.scale,
                            splits, self._scratch if splits > 1 else None, out_tpad=ht.t_pad, sparse_idx=sel)
        self._unabsorb(L, T, small, o_slab, ht)
        self.launches += (7 if small else 8) + (1 if splits > 1 else 0)

    def _unabsorb(self, L, T: int, small: bool, o_slab: torch.Tensor, ht) -> None:
        """Latent attention output -> per-head values through W_uv, then the o projection with the residual add."""
        ws = self.ws
        if small:
            K.mla_unabsorb_small(o_slab, L.w_uv, ws.attn[:T], T)
        else:
            K.grouped_linear(o_slab.view(-1, 512), L.w_uv, ws.attn, ht.tile_expert, ht.tile_row0, ht.num_tiles, ht.max_tiles,
                             ht.tile_rows, row_dst=ht.row_dst, ldo=self.cfg.v_head_dim, split_k=False)
        self._proj_o(L, T)

    # The two ends of the attention half that a tensor-parallel engine replaces (models/tp_mla.py): where the
    # normalised rows come from, and where the o projection's output goes.
    def _x_rows(self, T: int) -> torch.Tensor:
        return self.ws.x[:T]

    def _proj_a(self, L, T: int) -> None:
        K.linear(self.ws.x[:T], L.wqkv_a, out=self.ws.a[:T])

    def _proj_o(self, L, T: int, twin: bool = True) -> None:
        ws = self.ws
        if twin:
            self._linear(L, "wo", ws.attn[:T], ws.h[:T], residual=ws.h[:T])
        else:
            K.linear(ws.attn[:T], L.wo, out=ws.h[:T], residual=ws.h[:T])

    def _select(self, i: int, T: int, b: Batch) -> torch.Tensor:
        """Lightning indexer: store this step's index keys, score every visible position, keep the top-k per token."""
        cfg, L, ws = self.cfg, self.W.layers[i], self.ws
        Hi, off_k = cfg.indexer_heads, cfg.q_lora_rank + REC
        off_w = off_k + cfg.indexer_dim
        S, max_pages = b.page_table.shape
        ld = ((max_pages * PAGE + 127) // 128) * 128
        if ws.scores is None or ws.scores.shape[1] < ld:
            ws.scores = torch.empty(self.max_tokens, ld, dtype=torch.float32, device=self.device)
        K.index_k_store(ws.a[:T, off_k:off_w], b.slots, self.kv.idx[i])
        K.linear(ws.x[:T], L.wq_idx, out=ws.q_idx[:T])
        ibs, ibt = self._block_table(S, b.max_q_len, 256 // Hi)
        tiles = (max_pages + 1) // 2
        splits = 1 if b.prefill else max(1, min(K.num_sms() // max(1, ibs.numel()), max(1, tiles // 2), 64))
        K.indexer_scores(ws.q_idx[:T].view(T, Hi, cfg.indexer_dim), self.kv.idx[i], ws.a[:T, off_w:off_w + Hi], b.page_table,
                         b.seq_lens, b.q_start, ibs, ibt, ws.scores[:T], splits, w_scale=Hi ** -0.5)
        K.index_topk(ws.scores[:T], cfg.indexer_topk, ws.sel[:T], seq_lens=b.seq_lens, q_start=b.q_start)
        self.launches += 4
        if self.select_hook is not None:
            self.select_hook(i, ws.sel[:T])
        return ws.sel[:T]
