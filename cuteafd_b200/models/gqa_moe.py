"""GQA + MoE decoder (Qwen3-MoE geometry and relatives) on the sm_100a kernels.

Weights are held in the layout the kernels stream: fused qkv rows, per-layer stacked expert
tensors [E, I, H] / [E, H, I].  Stacking copies rows; it re-encodes nothing.  The forward pass is
a fixed launch sequence over preallocated workspaces, so a decode step can be captured in a CUDA
graph.  The layer body mirrors the reference's per-layer segment
(rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2110-2262: norm -> attention unit ->
exchange -> post norm -> dense FFN or moe_front / moe_exchange), minus the host transport.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..config import ModelConfig
from ..ops import kernels as K
from ..parallel.moe_exchange import ExchangeGeometry, LocalExchange, pick_tile_rows

PAGE = 64


@dataclass
class Batch:
    """Device-side description of one forward step (all int32 tensors on the GPU)."""
    tokens: torch.Tensor        # [T]
    positions: torch.Tensor     # [T]
    slots: torch.Tensor         # [T] page * 64 + offset for the KV write
    page_table: torch.Tensor    # [S, max_pages]
    seq_lens: torch.Tensor      # [S] kv length after this step
    q_start: torch.Tensor       # [S + 1]
    max_q_len: int
    prefill: bool
    last_rows: torch.Tensor | None = None   # rows whose logits are wanted (None = all)
    fresh: bool = False                     # prefill of a single sequence from position 0 (no earlier context in the cache)
    # media rows: (row indices int64 [m], embeddings [m, hidden] bf16), both on the device; those rows of the input
    # take the tower's output instead of the embedding table's row (eager prefill only)
    embeds: tuple | None = None


class LayerWeights:
    # ``fp8``: optional {projection name: (E4M3 values [N, K], fp32 128x128 block scales)} twins of the bf16 projections,
    # used for decode-sized steps (``GqaMoeEngine._linear``)
    __slots__ = ("ln1", "ln2", "wqkv", "wo", "q_norm", "k_norm", "router", "router_bias", "w_gate", "w_up", "w_down",
                 "d_gate", "d_up", "d_down", "s_gate", "s_up", "s_down", "fp8", "bqkv")

    def __init__(self) -> None:
        for s in self.__slots__:
            setattr(self, s, None)


@dataclass
class MtpExtras:
    """What one multi-token-prediction depth adds around its decoder layer: the two input norms, the projection of
    [norm(embed(x_{t+1})) | norm(h_t)] split into its two column halves, and the norm before the shared head."""
    enorm: torch.Tensor
    hnorm: torch.Tensor
    w_e: torch.Tensor        # eh_proj[:, :H]
    w_h: torch.Tensor        # eh_proj[:, H:]
    head_norm: torch.Tensor


def layer_is_moe(cfg: ModelConfig, i: int) -> bool:
    return cfg.is_moe_layer(i) if i < cfg.num_layers else cfg.num_experts > 0


def load_mtp_extras(cfg: ModelConfig, p: dict, t) -> list[MtpExtras]:
    out = []
    H = cfg.hidden
    for j in range(cfg.mtp_layers):
        pre = f"model.layers.{cfg.num_layers + j}."
        if pre + "eh_proj.weight" not in p:
            break
        eh = t(pre + "eh_proj.weight")
        out.append(MtpExtras(t(pre + "enorm.weight"), t(pre + "hnorm.weight"), eh[:, :H].contiguous(), eh[:, H:].contiguous(),
                             t(pre + "shared_head.norm.weight")))
    return out


class GqaMoeWeights:
    def __init__(self, cfg: ModelConfig):
        self.cfg = cfg
        self.embed: torch.Tensor | None = None
        self.final_norm: torch.Tensor | None = None
        self.lm_head: torch.Tensor | None = None
        self.layers: list[LayerWeights] = []
        self.mtp: list[MtpExtras] = []

    @staticmethod
    def from_params(cfg: ModelConfig, p: dict[str, torch.Tensor], device: torch.device,
                    with_experts: bool = True) -> "GqaMoeWeights":
        """Build from a Hugging Face style name -> tensor dictionary (any float dtype).
        ``with_experts=False`` leaves the routed experts out (they live on expert ranks)."""
        def t(name: str) -> torch.Tensor:
            return p[name].to(device=device, dtype=torch.bfloat16).contiguous()

        W = GqaMoeWeights(cfg)
        W.embed, W.final_norm = t("model.embed_tokens.weight"), t("model.norm.weight")
        W.lm_head = W.embed if cfg.tie_embeddings else t("lm_head.weight")
        W.mtp = load_mtp_extras(cfg, p, t)
        for i in range(cfg.num_layers + cfg.mtp_layers):     # MTP decoder layers follow the main stack
            pre, L = f"model.layers.{i}.", LayerWeights()
            a, m = pre + "self_attn.", pre + "mlp."
            L.ln1, L.ln2 = t(pre + "input_layernorm.weight"), t(pre + "post_attention_layernorm.weight")
            L.wqkv = torch.cat([t(a + "q_proj.weight"), t(a + "k_proj.weight"), t(a + "v_proj.weight")]).contiguous()
            if cfg.attention_bias:
                L.bqkv = torch.cat([t(a + "q_proj.bias"), t(a + "k_proj.bias"), t(a + "v_proj.bias")]).contiguous()
            L.wo = t(a + "o_proj.weight")
            if cfg.qk_norm:
                L.q_norm, L.k_norm = t(a + "q_norm.weight"), t(a + "k_norm.weight")
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
                    with_experts: bool = True) -> "GqaMoeWeights":
        """N(0, std) weights generated on the device, layer by layer (no host copy of the model)."""
        g = torch.Generator(device=device).manual_seed(seed)

        def w(*shape: int) -> torch.Tensor:
            out = torch.empty(*shape, dtype=torch.bfloat16, device=device)
            out.normal_(0.0, std, generator=g)
            return out

        def ones(n: int) -> torch.Tensor:
            return torch.ones(n, dtype=torch.bfloat16, device=device)

        H, D = cfg.hidden, cfg.head_dim
        W = GqaMoeWeights(cfg)
        W.embed, W.final_norm = w(cfg.vocab_size, H), ones(H)
        W.lm_head = W.embed if cfg.tie_embeddings else w(cfg.vocab_size, H)
        W.mtp = [MtpExtras(ones(H), ones(H), w(H, H), w(H, H), ones(H)) for _ in range(cfg.mtp_layers)]
        for i in range(cfg.num_layers + cfg.mtp_layers):
            L = LayerWeights()
            L.ln1, L.ln2 = ones(H), ones(H)
            L.wqkv, L.wo = w((cfg.num_heads + 2 * cfg.num_kv_heads) * D, H), w(H, cfg.num_heads * D)
            if cfg.attention_bias:
                L.bqkv = w((cfg.num_heads + 2 * cfg.num_kv_heads) * D)
            if cfg.qk_norm:
                L.q_norm, L.k_norm = ones(D), ones(D)
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


class KvCache:
    """Paged K/V pools, one pair per layer: [num_pages, Hkv, 64, D] bf16 (the tile of one page and kv head is 16 KB of
    contiguous memory: decode attention streams whole tiles).  Page 0 stays all-zero:
    kernels read it for table entries past a sequence's end (the reference keeps the same
    reserved page, rust/crates/cuteafd-engine/src/prefix/family.rs:20-28)."""

    def __init__(self, cfg: ModelConfig, num_pages: int, device: torch.device):
        shape = (num_pages, cfg.num_kv_heads, PAGE, cfg.head_dim)     # one (page, head) tile is contiguous
        self.num_pages = num_pages
        n = cfg.num_layers + cfg.mtp_layers              # MTP decoder layers keep their own K/V, same pages
        self.k = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(n)]
        self.v = [torch.zeros(shape, dtype=torch.bfloat16, device=device) for _ in range(n)]

    def bytes_per_page(self) -> int:
        return 2 * len(self.k) * self.k[0][0].numel() * 2

    def copy_page(self, src: int, dst: int) -> None:
        for k, v in zip(self.k, self.v):
            k[dst].copy_(k[src])
            v[dst].copy_(v[src])


class Workspace:
    def __init__(self, cfg: ModelConfig, max_tokens: int, device: torch.device):
        H, D = cfg.hidden, cfg.head_dim
        bf = dict(dtype=torch.bfloat16, device=device)
        self.h = torch.empty(max_tokens, H, **bf)
        self.x = torch.empty(max_tokens, H, **bf)
        self.qkv = torch.empty(max_tokens, (cfg.num_heads + 2 * cfg.num_kv_heads) * D, **bf)
        self.q = torch.empty(max_tokens, cfg.num_heads, D, **bf)
        self.attn = torch.empty(max_tokens, cfg.num_heads, D, **bf)
        self.router = torch.empty(max_tokens, max(cfg.num_experts, 1), dtype=torch.float32, device=device)
        dense = cfg.first_dense_layers > 0 or cfg.num_experts == 0
        self.ffn_d = torch.empty(max_tokens, cfg.dense_ffn, **bf) if dense else None
        self.ffn_s = torch.empty(max_tokens, cfg.expert_ffn * cfg.num_shared_experts, **bf) if cfg.num_shared_experts else None
        self.shared = torch.empty(max_tokens, H, **bf) if cfg.num_shared_experts else None


class GqaMoeEngine:
    """Single-GPU engine (attention and experts on the same device)."""
    fused = None                 # class defaults: subclasses with their own constructor never take the fused step
    _fused_rows = 0
    _fused_checked = False
    embed_rows = None            # [max_tokens, hidden] staging of a host-resident embedding table's rows (None = table on the GPU)

    def __init__(self, cfg: ModelConfig, weights: GqaMoeWeights, kv: KvCache, max_tokens: int, max_seqs: int = 64,
                 build_moe: bool = True):
        assert cfg.attention == "gqa" and cfg.head_dim == 128
        self.cfg, self.W, self.kv = cfg, weights, kv
        self.device = weights.embed.device
        self.max_tokens = max_tokens
        self.ws = Workspace(cfg, max_tokens, self.device)
        from ..ref.ops import rope_inv_freq, rope_magnitudes
        if rope_magnitudes(cfg) != (1.0, 1.0):
            # the GQA attention kernels take no softmax-scale argument and the rope kernel no magnitude
            raise ValueError("YaRN magnitude scaling is not supported by the GQA engine (linear and llama3 scaling are)")
        self.inv_freq = rope_inv_freq(cfg, cfg.rope_dim).to(self.device)      # long-context scaling is in this table
        self.moe = None
        self.pre_moe = None          # hook(layer) called before each MoE layer's exchange
        if cfg.num_experts and build_moe:
            geo = ExchangeGeometry(cfg.hidden, cfg.expert_ffn, cfg.num_experts, cfg.top_k, max_tokens, 1)
            self.moe = LocalExchange(geo, self.device)
        self.route_kw = dict(scoring=cfg.scoring, num_groups=cfg.num_groups, topk_groups=cfg.topk_groups,
                             normalize=cfg.norm_topk_prob, routed_scale=cfg.routed_scale)
        self.logits = torch.empty(max_seqs if max_seqs < max_tokens else max_tokens, cfg.vocab_size,
                                  dtype=torch.float32, device=self.device)
        self.next_tokens = torch.empty(self.logits.shape[0], dtype=torch.int32, device=self.device)
        self._scratch: torch.Tensor | None = None
        self.fixed_kv_split = K.batch_invariant_from_env()     # tokens per kv split in the batch-invariant form, else 0
        self.launches = 0
        self._f8_rows = {}
        # one-launch decode step (ops/decode_step.py): built lazily for the geometries it takes, single-GPU experts only
        self.fused = None
        self._fused_rows = 0
        self._fused_checked = False

    # ---- one-launch decode step -------------------------------------------------------------------
    def _fused_for(self, b: Batch):
        """The fused decode step when batch ``b`` is a plain decode step it can run, else None."""
        if b.prefill or b.max_q_len != 1 or b.last_rows is not None or b.embeds is not None:
            return None
        if not self._fused_checked:
            self._fused_checked = True
            from ..ops.decode_step import FusedDecodeStep
            if (type(self) is GqaMoeEngine and isinstance(self.moe, LocalExchange) and FusedDecodeStep.supports(self.cfg)
                    and self.W.layers[0].w_gate is not None and getattr(self.W, "expert_format", "bf16") == "bf16"
                    and self.device.type == "cuda"):
                self.fused = FusedDecodeStep(self)
        if self.fused is None or b.tokens.shape[0] > self.fused.MAX_ROWS or b.page_table.shape[0] != b.tokens.shape[0]:
            return None
        return self.fused

    def decode_step(self, b: Batch, advance: bool = False) -> torch.Tensor:
        """Forward + greedy selection of one decode step; with ``advance`` the batch's token / position / length /
        slot vectors are moved to the next step on the device.  Returns the selected tokens."""
        f = self._fused_for(b)
        if f is not None:
            _, nxt = f.run(b, advance=advance)
            self.launches += 1
            return nxt
        out = self.greedy(self.forward(b))
        if advance:
            K.decode_advance(b.tokens, out, b.positions, b.seq_lens, b.slots, b.page_table)
            self.launches += 1
        return out

    # ---- pieces ---------------------------------------------------------------------------------
    def _attention(self, i: int, T: int, b: Batch) -> None:
        cfg, L, ws = self.cfg, self.W.layers[i], self.ws
        K.linear(ws.x[:T], L.wqkv, out=ws.qkv[:T])
        K.qk_rope_kv(ws.qkv[:T], L.q_norm, L.k_norm, self.inv_freq, b.positions, b.slots, ws.q[:T], self.kv.k[i],
                     self.kv.v[i], cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rms_eps, cfg.rope_interleaved,
                     bias=L.bqkv)
        if b.prefill:
            K.attn_prefill(ws.q[:T], self.kv.k[i], self.kv.v[i], b.page_table, b.seq_lens, b.q_start, ws.attn[:T],
                           b.max_q_len, window=cfg.window_of(i))
            self.launches += 3
        else:
            S, max_pages = b.page_table.shape
            q_per_tile = 16 // (cfg.num_heads // cfg.num_kv_heads)
            tiles = (b.max_q_len + q_per_tile - 1) // q_per_tile
            splits = K.kv_splits_fixed(max_pages) if self.fixed_kv_split else K.attn_decode_splits(S, tiles, cfg.num_kv_heads, max_pages, cfg.window_of(i))
            need = K.attn_decode_scratch_floats(S, b.max_q_len, cfg.num_heads, cfg.num_kv_heads, splits)
            if self._scratch is None or self._scratch.numel() < need:
                self._scratch = torch.empty(need, dtype=torch.float32, device=self.device)
            K.attn_decode(ws.q[:T], self.kv.k[i], self.kv.v[i], b.page_table, b.seq_lens, b.q_start, ws.attn[:T],
                          self._scratch, b.max_q_len, splits, window=cfg.window_of(i))
            self.launches += 3 + (1 if splits > 1 else 0)
        # o_proj with the residual add fused into the epilogue: h = h + attn @ wo.T
        K.linear(ws.attn[:T].view(T, -1), L.wo, out=ws.h[:T], residual=ws.h[:T])
        self.launches += 1

    FUSED_ROUTE_TOKENS = 64         # steps up to this many tokens run RMSNorm + router + top-k as one launch
    FP8_LINEAR_TOKENS = 64          # steps up to this many tokens take a projection's E4M3 twin when the layer has one

    def _linear(self, L, name: str, x: torch.Tensor, out: torch.Tensor, *, up: str | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
        """``out = x @ L.<name>.T`` (SwiGLU pair with ``up``).  Decode-sized steps of a layer that carries E4M3 twins
        (``L.fp8``) quantise the rows 1x128 and run the block-scaled GEMM: the step streams half the weight bytes
        (DeepSeek-V3 o projection at 8 rows: 48.1 -> 38.3 us with the quantise launch, q_b 22.5 -> 18.0, shared expert
        18.6 + 13.7 -> 16.4 + 11.3).  Larger steps stay on the bf16 weights, where the bf16 kernel is the faster one."""
        T = x.shape[0]
        f8 = getattr(L, "fp8", None)
        if f8 and name in f8 and T <= self.FP8_LINEAR_TOKENS:
            Kd = x.shape[1]
            buf = self._f8_rows.get(Kd)
            if buf is None:
                buf = (torch.empty(self.FP8_LINEAR_TOKENS, Kd, dtype=torch.float8_e4m3fn, device=self.device),
                       torch.empty(self.FP8_LINEAR_TOKENS, Kd // 128, dtype=torch.float32, device=self.device))
                self._f8_rows[Kd] = buf
            xq, xs = buf[0][:T], buf[1][:T]
            K.quant_rows_fp8(x, xq, xs)
            w, u = f8[name], (f8[up] if up else None)
            self.launches += 1
            return K.linear_fp8(xq, xs, w[0], w[1], out, w_up=u[0] if u else None, ws_up=u[1] if u else None, residual=residual)
        return K.linear(x, getattr(L, name), out=out, w_up=getattr(L, up) if up else None, residual=residual)

    def _exchange_launches(self, T: int) -> int:
        """Kernels one bf16 exchange launches for T tokens: plan (with the dispatch folded in for very small steps, three
        launches wide from 8192 entries on), dispatch, fc1, fc2, combine."""
        from ..parallel.moe_exchange import AttentionSide as A
        n = T * self.cfg.top_k
        fused = n <= A.FUSED_DISPATCH_ROWS and n * self.cfg.hidden * 2 <= A.FUSED_DISPATCH_BYTES
        return (4 if fused else 5) + (2 if n >= K.WIDE_PLAN_ENTRIES else 0)

    def _ffn(self, i: int, T: int, next_norm: torch.Tensor | None) -> bool:
        """Post-attention norm + FFN of layer i.  Returns True when ``ws.x`` already holds the next layer's
        normalised input (the MoE combine fused that norm in)."""
        cfg, L, ws = self.cfg, self.W.layers[i], self.ws
        if L.router is None:
            K.rmsnorm(ws.h[:T], L.ln2, cfg.rms_eps, out=ws.x[:T])
            K.linear(ws.x[:T], L.d_gate, out=ws.ffn_d[:T], w_up=L.d_up)
            K.linear(ws.ffn_d[:T], L.d_down, out=ws.h[:T], residual=ws.h[:T])
            self.launches += 3
            return False
        fused = T <= self.FUSED_ROUTE_TOKENS and cfg.hidden <= 8192 and hasattr(self.moe, "att")
        logits = None
        if fused:
            K.norm_route(ws.h[:T], L.ln2, cfg.rms_eps, L.router, ws.x[:T], self.moe.att.idx[:T], self.moe.att.w[:T], cfg.top_k,
                         bias=L.router_bias, **self.route_kw)
            self.launches += 1
        else:
            K.rmsnorm(ws.h[:T], L.ln2, cfg.rms_eps, out=ws.x[:T])
            logits = K.linear(ws.x[:T], L.router, out=ws.router[:T, :cfg.num_experts], out_f32=True)
            self.launches += 3                   # norm, router scores, top-k
        kw = dict(self.route_kw, bias=L.router_bias)
        if self.pre_moe is not None:
            self.pre_moe(i)
        split = hasattr(self.moe, "begin")
        if split:
            # disaggregated exchange: the rows leave for the expert ranks first, the shared expert's GEMMs run while
            # they are away, the combine waits for them last
            self.moe.begin(ws.x[:T], logits, kw)
        shared = None
        if L.s_gate is not None:
            self._linear(L, "s_gate", ws.x[:T], ws.ffn_s[:T], up="s_up")
            shared = self._linear(L, "s_down", ws.ffn_s[:T], ws.shared[:T])
            self.launches += 2
        if split:
            self.moe.finish(ws.h[:T], shared=shared, residual=ws.h[:T], norm_w=next_norm, eps=cfg.rms_eps,
                            x_out=ws.x[:T] if next_norm is not None else None)
            self.launches += self._exchange_launches(T)
            return next_norm is not None
        fmt = getattr(self.W, "expert_format", "bf16")
        if fmt != "bf16" and hasattr(self.moe, "forward_stored"):
            # experts served in their stored form (E4M3 block-scaled / MXFP4 / NVFP4): same exchange, quantised GEMMs
            self.moe.forward_stored(fmt, ws.x[:T], logits, kw, L.w_gate, L.w_up, L.w_down, ws.h[:T], shared=shared,
                                    residual=ws.h[:T])
            self.launches += 6
            return False
        self.moe.forward(ws.x[:T], logits, kw, L.w_gate, L.w_up, L.w_down, ws.h[:T], shared=shared, residual=ws.h[:T],
                         norm_w=next_norm, eps=cfg.rms_eps, x_out=ws.x[:T] if next_norm is not None else None)
        self.launches += self._exchange_launches(T)             # plan(+dispatch), fc1, fc2, combine
        return next_norm is not None

    # ---- whole step -------------------------------------------------------------------------------
    def forward(self, b: Batch) -> torch.Tensor:
        """Runs all layers; returns fp32 logits for ``b.last_rows`` (or every row)."""
        cfg, ws = self.cfg, self.ws
        T = b.tokens.shape[0]
        assert T <= self.max_tokens
        self._fused_rows = 0
        f = self._fused_for(b)
        if f is not None:
            logits, _ = f.run(b)
            self.launches += 1
            self._fused_rows = T             # ``greedy`` on these logits returns the tokens the step already selected
            return logits
        if self.embed_rows is not None:
            # host-resident embedding table: the backend gathered this step's rows from the memory-mapped table and
            # staged them in ``embed_rows`` (a fixed buffer, so captured graphs read it too)
            ws.h[:T].copy_(self.embed_rows[:T])
        else:
            K.embed(b.tokens, self.W.embed, out=ws.h[:T])
        self.launches += 1
        if b.embeds is not None:
            ws.h[:T].index_copy_(0, b.embeds[0], b.embeds[1])
        have_x = False
        for i in range(cfg.num_layers):
            L = self.W.layers[i]
            if not have_x:
                K.rmsnorm(ws.h[:T], L.ln1, cfg.rms_eps, out=ws.x[:T])
                self.launches += 1
            self._attention(i, T, b)
            nxt = self.W.layers[i + 1].ln1 if i + 1 < cfg.num_layers else None
            have_x = self._ffn(i, T, nxt)
        if b.last_rows is not None:
            rows = ws.h[:T].index_select(0, b.last_rows)
        else:
            rows = ws.h[:T]
        n = rows.shape[0]
        xn = K.rmsnorm(rows, self.W.final_norm, cfg.rms_eps, out=ws.x[:n])
        logits = K.linear(xn, self.W.lm_head, out=self.logits[:n], out_f32=True)
        self.launches += 2
        return logits

    # ---- multi-token prediction ---------------------------------------------------------------------
    def mtp_forward(self, j: int, b: Batch, next_tokens: torch.Tensor) -> torch.Tensor:
        """MTP depth j right after ``forward(b)``: row t pairs the backbone's final hidden state of position t (still
        in the workspace) with ``next_tokens[t]`` (the token that follows it), runs the depth's decoder layer with its
        own K/V at the same positions and pages, and returns fp32 logits predicting the token after next for every row
        (python/reference/families/qwen4/mtp.py:1-32; speculation/recurrent.rs:18-40 in the reference daemon)."""
        cfg, ws, X = self.cfg, self.ws, self.W.mtp[j]
        li = cfg.num_layers + j
        T = b.tokens.shape[0]
        if getattr(ws, "mtp_e", None) is None:
            bf = dict(dtype=torch.bfloat16, device=self.device)
            ws.mtp_e, ws.mtp_t = torch.empty(self.max_tokens, cfg.hidden, **bf), torch.empty(self.max_tokens, cfg.hidden, **bf)
            self.mtp_logits = torch.empty(min(self.max_tokens, max(256, self.logits.shape[0] * 8)), cfg.vocab_size, dtype=torch.float32,
                                          device=self.device)
        K.rmsnorm(ws.h[:T], X.hnorm, cfg.rms_eps, out=ws.mtp_t[:T])                 # h_t before it is overwritten
        K.embed(next_tokens, self.W.embed, out=ws.mtp_e[:T])
        K.rmsnorm(ws.mtp_e[:T], X.enorm, cfg.rms_eps, out=ws.x[:T])
        K.linear(ws.x[:T], X.w_e, out=ws.mtp_e[:T])
        K.linear(ws.mtp_t[:T], X.w_h, out=ws.h[:T], residual=ws.mtp_e[:T])          # eh_proj([e | h]) as two halves
        K.rmsnorm(ws.h[:T], self.W.layers[li].ln1, cfg.rms_eps, out=ws.x[:T])
        self._attention(li, T, b)
        self._ffn(li, T, None)
        n = min(T, self.mtp_logits.shape[0])
        K.rmsnorm(ws.h[:n], X.head_norm, cfg.rms_eps, out=ws.x[:n])
        self.launches += 8
        return K.linear(ws.x[:n], self.W.lm_head, out=self.mtp_logits[:n], out_f32=True)

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        if self._fused_rows and self._fused_rows == logits.shape[0] and logits.data_ptr() == self.logits.data_ptr():
            return self.next_tokens[:logits.shape[0]]
        self.launches += 1
        return K.argmax(logits, out=self.next_tokens[:logits.shape[0]])
