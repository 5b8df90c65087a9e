"""CPU oracle decoder: every family the engine serves, in readable PyTorch.

It is the numerics oracle for the CUDA engine, the timed CPU baseline, and the "whole" side of
the whole-versus-split test (one attention rank plus expert ranks over gloo).  Parameter names
follow the Hugging Face snapshot layout so the same dictionary can be written to and read from
safetensors shards.  The reference's per-family goldens work the same way, one layer at a time
(python/reference/layer_major.py:1-22, python/reference/cuteafd_reference/layer_ref.py:12-36).
"""
from __future__ import annotations

import math
from typing import Callable

import torch

from ..config import ModelConfig
from . import ops

MoeFn = Callable[[int, torch.Tensor, torch.Tensor, torch.Tensor], torch.Tensor]


def init_weights(cfg: ModelConfig, seed: int = 0, dtype: torch.dtype = torch.float32, std: float = 0.02,
                 device: str = "cpu") -> dict[str, torch.Tensor]:
    """Random-init parameters N(0, std), norm weights one, router bias zero."""
    g = torch.Generator(device="cpu").manual_seed(seed)

    def w(*shape: int) -> torch.Tensor:
        return (torch.randn(*shape, generator=g) * std).to(dtype).to(device)

    def ones(n: int) -> torch.Tensor:
        return torch.ones(n, dtype=dtype, device=device)

    H = cfg.hidden
    p: dict[str, torch.Tensor] = {"model.embed_tokens.weight": w(cfg.vocab_size, H), "model.norm.weight": ones(H)}
    if not cfg.tie_embeddings:
        p["lm_head.weight"] = w(cfg.vocab_size, H)
    n_layers = cfg.num_layers + cfg.mtp_layers
    for i in range(n_layers):
        pre = f"model.layers.{i}."
        p[pre + "input_layernorm.weight"] = ones(H)
        p[pre + "post_attention_layernorm.weight"] = ones(H)
        a = pre + "self_attn."
        if cfg.is_mla:
            qd = cfg.num_heads * cfg.qk_head_dim
            if cfg.q_lora_rank:
                p[a + "q_a_proj.weight"] = w(cfg.q_lora_rank, H)
                p[a + "q_a_layernorm.weight"] = ones(cfg.q_lora_rank)
                p[a + "q_b_proj.weight"] = w(qd, cfg.q_lora_rank)
            else:
                p[a + "q_proj.weight"] = w(qd, H)
            p[a + "kv_a_proj_with_mqa.weight"] = w(cfg.kv_lora_rank + cfg.qk_rope_dim, H)
            p[a + "kv_a_layernorm.weight"] = ones(cfg.kv_lora_rank)
            p[a + "kv_b_proj.weight"] = w(cfg.num_heads * (cfg.qk_nope_dim + cfg.v_head_dim), cfg.kv_lora_rank)
            p[a + "o_proj.weight"] = w(H, cfg.num_heads * cfg.v_head_dim)
            if cfg.indexer_heads:
                p[a + "indexer.wq.weight"] = w(cfg.indexer_heads * cfg.indexer_dim, H)
                p[a + "indexer.wk.weight"] = w(cfg.indexer_dim, H)
                p[a + "indexer.weights_proj.weight"] = w(cfg.indexer_heads, H)
        else:
            p[a + "q_proj.weight"] = w(cfg.num_heads * cfg.head_dim, H)
            p[a + "k_proj.weight"] = w(cfg.num_kv_heads * cfg.head_dim, H)
            p[a + "v_proj.weight"] = w(cfg.num_kv_heads * cfg.head_dim, H)
            p[a + "o_proj.weight"] = w(H, cfg.num_heads * cfg.head_dim)
            if cfg.attention_bias:
                for n, rows in (("q", cfg.num_heads), ("k", cfg.num_kv_heads), ("v", cfg.num_kv_heads)):
                    p[a + f"{n}_proj.bias"] = w(rows * cfg.head_dim)
            if cfg.qk_norm:
                p[a + "q_norm.weight"] = ones(cfg.head_dim)
                p[a + "k_norm.weight"] = ones(cfg.head_dim)
        m = pre + "mlp."
        moe = cfg.is_moe_layer(i) if i < cfg.num_layers else cfg.num_experts > 0
        if moe:
            p[m + "gate.weight"] = w(cfg.num_experts, H)
            if cfg.router_bias:
                p[m + "gate.e_score_correction_bias"] = torch.zeros(cfg.num_experts, dtype=torch.float32, device=device)
            for e in range(cfg.num_experts):
                p[m + f"experts.{e}.gate_proj.weight"] = w(cfg.expert_ffn, H)
                p[m + f"experts.{e}.up_proj.weight"] = w(cfg.expert_ffn, H)
                p[m + f"experts.{e}.down_proj.weight"] = w(H, cfg.expert_ffn)
            if cfg.num_shared_experts:
                inter = cfg.expert_ffn * cfg.num_shared_experts
                p[m + "shared_experts.gate_proj.weight"] = w(inter, H)
                p[m + "shared_experts.up_proj.weight"] = w(inter, H)
                p[m + "shared_experts.down_proj.weight"] = w(H, inter)
        else:
            p[m + "gate_proj.weight"] = w(cfg.dense_ffn, H)
            p[m + "up_proj.weight"] = w(cfg.dense_ffn, H)
            p[m + "down_proj.weight"] = w(H, cfg.dense_ffn)
        if i >= cfg.num_layers:                       # MTP layer extras (DeepSeek-V3 layout)
            p[pre + "enorm.weight"] = ones(H)
            p[pre + "hnorm.weight"] = ones(H)
            p[pre + "eh_proj.weight"] = w(H, 2 * H)
            p[pre + "shared_head.norm.weight"] = ones(H)
    return p


class KvState:
    """Per-sequence, per-layer cached rows: latent+rope for MLA, (k, v) for GQA."""

    def __init__(self, cfg: ModelConfig):
        n = cfg.num_layers + cfg.mtp_layers
        self.rows: list[list[torch.Tensor]] = [[] for _ in range(n)]

    def length(self, layer: int = 0) -> int:
        return sum(r.shape[0] for r in self.rows[layer])

    def append(self, layer: int, rec: torch.Tensor) -> torch.Tensor:
        self.rows[layer].append(rec)
        full = torch.cat(self.rows[layer], dim=0)
        self.rows[layer] = [full]
        return full

    def truncate(self, length: int) -> None:
        for i, r in enumerate(self.rows):
            if r:
                self.rows[i] = [torch.cat(r, dim=0)[:length]]


class RefDecoder:
    """Functional decoder over a parameter dictionary.  ``moe_fn`` replaces the routed-expert
    computation (used by the split run to send the work to expert ranks)."""

    def __init__(self, cfg: ModelConfig, params: dict[str, torch.Tensor], moe_fn: MoeFn | None = None):
        self.cfg, self.p, self.moe_fn = cfg, params, moe_fn
        self.select_fn = None        # optional (layer, start, Tq, Tk) -> bool mask [Tq, Tk] replacing the indexer's choice
        self.inv_freq = ops.rope_inv_freq(cfg, cfg.rope_dim)        # long-context scaling lives in this table
        self.rope_mag, self.scale_mul = ops.rope_magnitudes(cfg)
        self.usage: dict[int, torch.Tensor] | None = None     # set to {} to count routed tokens per layer and expert
        self.observe = None          # optional (operand prefix, input rows [n, in]) -> None, called before every projection
        self._stacked: dict[int, tuple[torch.Tensor, torch.Tensor, torch.Tensor]] = {}

    def _see(self, prefix: str, x: torch.Tensor) -> None:
        if self.observe is not None and x.shape[0]:
            self.observe(prefix, x)

    def _see_mlp(self, prefix: str, x: torch.Tensor) -> None:
        """Inputs of a SwiGLU block's three projections (the down projection sees the rounded activation)."""
        if self.observe is None or not x.shape[0]:
            return
        p = self.p
        self.observe(prefix + "gate_proj", x)
        self.observe(prefix + "up_proj", x)
        xf = x.float()
        act = torch.nn.functional.silu(xf @ p[prefix + "gate_proj.weight"].float().T) * (xf @ p[prefix + "up_proj.weight"].float().T)
        self.observe(prefix + "down_proj", act.to(x.dtype))

    # ---- pieces ---------------------------------------------------------------------------
    def expert_stack(self, layer: int, lo: int = 0, hi: int | None = None):
        hi = self.cfg.num_experts if hi is None else hi
        key = (layer, lo, hi)
        if key not in self._stacked:
            m = f"model.layers.{layer}.mlp.experts."
            self._stacked[key] = tuple(
                torch.stack([self.p[f"{m}{e}.{n}_proj.weight"] for e in range(lo, hi)]) for n in ("gate", "up", "down"))
        return self._stacked[key]

    def attention(self, layer: int, x: torch.Tensor, positions: torch.Tensor, kv: KvState) -> torch.Tensor:
        cfg, p = self.cfg, self.p
        a = f"model.layers.{layer}.self_attn."
        T = x.shape[0]
        start = int(positions[0])
        if self.observe is not None:
            for name in ("q_a_proj", "q_proj", "kv_a_proj_with_mqa", "k_proj", "v_proj", "indexer.wk", "indexer.wq",
                         "indexer.weights_proj"):
                if a + name + ".weight" in p:
                    self._see(a + name, x)
        if cfg.is_mla:
            if cfg.q_lora_rank:
                qa = ops.rmsnorm((x.float() @ p[a + "q_a_proj.weight"].float().T).to(x.dtype),
                                 p[a + "q_a_layernorm.weight"], cfg.rms_eps)
                self._see(a + "q_b_proj", qa)
                q = (qa.float() @ p[a + "q_b_proj.weight"].float().T).to(x.dtype)
            else:
                q = (x.float() @ p[a + "q_proj.weight"].float().T).to(x.dtype)
            q = q.view(T, cfg.num_heads, cfg.qk_head_dim)
            q_nope, q_rope = q[..., : cfg.qk_nope_dim], q[..., cfg.qk_nope_dim:]
            q_rope = ops.apply_rope(q_rope, positions, cfg.rope_theta, cfg.rope_interleaved, self.inv_freq, self.rope_mag)
            ckv = (x.float() @ p[a + "kv_a_proj_with_mqa.weight"].float().T).to(x.dtype)
            latent = ops.rmsnorm(ckv[:, : cfg.kv_lora_rank], p[a + "kv_a_layernorm.weight"], cfg.rms_eps)
            k_rope = ops.apply_rope(ckv[:, None, cfg.kv_lora_rank:], positions, cfg.rope_theta, cfg.rope_interleaved,
                                    self.inv_freq, self.rope_mag)[:, 0]
            if cfg.kv_format == "fp8_ds_mla":
                latent = ops.fp8_latent_roundtrip(latent)          # what the 656-byte record keeps of the latents
            rec = [latent, k_rope]
            if cfg.indexer_heads:
                rec.append((x.float() @ p[a + "indexer.wk.weight"].float().T).to(x.dtype))
            full = kv.append(layer, torch.cat(rec, dim=-1))
            lat_all, rope_all = full[:, : cfg.kv_lora_rank], full[:, cfg.kv_lora_rank: cfg.kv_lora_rank + cfg.qk_rope_dim]
            allowed = None
            if cfg.indexer_heads:
                # lightning indexer (simplified: no rope / rotation on the index vectors): index queries and
                # head weights from the layer input, index keys cached beside the latent record
                q_idx = (x.float() @ p[a + "indexer.wq.weight"].float().T).to(x.dtype).view(T, cfg.indexer_heads, cfg.indexer_dim)
                hw = (x.float() @ p[a + "indexer.weights_proj.weight"].float().T).to(x.dtype).float() * cfg.indexer_heads ** -0.5
                allowed = ops.index_select(q_idx, full[:, cfg.kv_lora_rank + cfg.qk_rope_dim:], hw, start, cfg.indexer_topk)
                if self.select_fn is not None:
                    forced = self.select_fn(layer, start, T, full.shape[0], allowed)
                    allowed = allowed if forced is None else forced
            self._see(a + "kv_b_proj", lat_all[-T:])
            kvb = (lat_all.float() @ p[a + "kv_b_proj.weight"].float().T).to(x.dtype)
            kvb = kvb.view(-1, cfg.num_heads, cfg.qk_nope_dim + cfg.v_head_dim)
            k = torch.cat([kvb[..., : cfg.qk_nope_dim], rope_all[:, None, :].expand(-1, cfg.num_heads, -1)], dim=-1)
            v = kvb[..., cfg.qk_nope_dim:]
            qq = torch.cat([q_nope, q_rope], dim=-1)
            o = ops.causal_attention(qq, k, v, start, self.scale_mul / math.sqrt(cfg.qk_head_dim), allowed)
            o = o.reshape(T, cfg.num_heads * cfg.v_head_dim)
        else:
            def proj(name: str, heads: int) -> torch.Tensor:
                y = (x.float() @ p[a + name + ".weight"].float().T).to(x.dtype)
                if cfg.attention_bias:       # projection rounded, bias added, rounded again (the engine adds it after the GEMM)
                    y = (y.float() + p[a + name + ".bias"].float()).to(x.dtype)
                return y.view(T, heads, cfg.head_dim)
            q, k, v = proj("q_proj", cfg.num_heads), proj("k_proj", cfg.num_kv_heads), proj("v_proj", cfg.num_kv_heads)
            if cfg.qk_norm:
                q = ops.rmsnorm(q, p[a + "q_norm.weight"], cfg.rms_eps)
                k = ops.rmsnorm(k, p[a + "k_norm.weight"], cfg.rms_eps)
            q = ops.apply_rope(q, positions, cfg.rope_theta, cfg.rope_interleaved, self.inv_freq, self.rope_mag)
            k = ops.apply_rope(k, positions, cfg.rope_theta, cfg.rope_interleaved, self.inv_freq, self.rope_mag)
            full = kv.append(layer, torch.cat([k.reshape(T, -1), v.reshape(T, -1)], dim=-1))
            half = cfg.num_kv_heads * cfg.head_dim
            k_all = full[:, :half].view(-1, cfg.num_kv_heads, cfg.head_dim)
            v_all = full[:, half:].view(-1, cfg.num_kv_heads, cfg.head_dim)
            o = ops.causal_attention(q, k_all, v_all, start, window=cfg.window_of(layer)).reshape(T, cfg.num_heads * cfg.head_dim)
        self._see(a + "o_proj", o)
        return (o.float() @ p[a + "o_proj.weight"].float().T).to(x.dtype)

    def route(self, layer: int, x: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        cfg, m = self.cfg, f"model.layers.{layer}.mlp."
        logits = x.float() @ self.p[m + "gate.weight"].float().T
        return ops.route_topk(logits, cfg.top_k, cfg.scoring, self.p.get(m + "gate.e_score_correction_bias"),
                              cfg.num_groups, cfg.topk_groups, cfg.norm_topk_prob, cfg.routed_scale)

    def ffn(self, layer: int, x: torch.Tensor, residual: torch.Tensor, moe: bool) -> torch.Tensor:
        """Returns the new residual stream: residual + ffn(x), rounded once."""
        p, m = self.p, f"model.layers.{layer}.mlp."
        if not moe:
            self._see_mlp(m, x)
            y = ops.swiglu_mlp(x, p[m + "gate_proj.weight"], p[m + "up_proj.weight"], p[m + "down_proj.weight"])
            return (residual.float() + y.to(x.dtype).float()).to(x.dtype)
        idx, w = self.route(layer, x)
        if self.usage is not None:                       # routed-token counts per layer and expert
            self.usage.setdefault(layer, torch.zeros(self.cfg.num_experts, dtype=torch.int64)).add_(
                torch.bincount(idx.reshape(-1), minlength=self.cfg.num_experts))
        if self.observe is not None:
            for e in idx.unique().tolist():
                self._see_mlp(f"{m}experts.{e}.", x[(idx == e).any(dim=-1)])
            if self.cfg.num_shared_experts:
                self._see_mlp(m + "shared_experts.", x)
        if self.moe_fn is not None:
            parts = self.moe_fn(layer, x, idx, w)
        else:
            parts = ops.moe_forward(x, idx, w, *self.expert_stack(layer))
        shared = None
        if self.cfg.num_shared_experts:
            s = m + "shared_experts."
            shared = ops.swiglu_mlp(x, p[s + "gate_proj.weight"], p[s + "up_proj.weight"],
                                    p[s + "down_proj.weight"]).to(x.dtype)
        return ops.combine_slots(parts, shared, residual, x.dtype)

    def layer(self, layer: int, h: torch.Tensor, positions: torch.Tensor, kv: KvState) -> torch.Tensor:
        cfg, p = self.cfg, self.p
        pre = f"model.layers.{layer}."
        x = ops.rmsnorm(h, p[pre + "input_layernorm.weight"], cfg.rms_eps)
        h = (h.float() + self.attention(layer, x, positions, kv).float()).to(h.dtype)
        x = ops.rmsnorm(h, p[pre + "post_attention_layernorm.weight"], cfg.rms_eps)
        moe = cfg.is_moe_layer(layer) if layer < cfg.num_layers else cfg.num_experts > 0
        return self.ffn(layer, x, h, moe)

    # ---- whole model ----------------------------------------------------------------------
    def embed(self, tokens: torch.Tensor) -> torch.Tensor:
        return self.p["model.embed_tokens.weight"][tokens]

    def head(self, h: torch.Tensor) -> torch.Tensor:
        x = ops.rmsnorm(h, self.p["model.norm.weight"], self.cfg.rms_eps)
        w = self.p["model.embed_tokens.weight"] if self.cfg.tie_embeddings else self.p["lm_head.weight"]
        return x.float() @ w.float().T

    def hidden_states(self, tokens: torch.Tensor, kv: KvState, embeds: tuple | None = None) -> torch.Tensor:
        """``embeds`` = (rows, values [m, hidden]): those input rows take ``values`` (media tower output) instead of
        the embedding table's row; their token ids may lie above the vocabulary."""
        start = kv.length(0)
        positions = torch.arange(start, start + tokens.shape[0], device=tokens.device)
        if embeds is not None:
            rows = torch.as_tensor(embeds[0], dtype=torch.long)
            tokens = tokens.clone()
            tokens[rows] = 0
            h = self.embed(tokens).clone()
            h[rows] = embeds[1].to(h.dtype)
        else:
            h = self.embed(tokens)
        for i in range(self.cfg.num_layers):
            h = self.layer(i, h, positions, kv)
        return h

    def forward(self, tokens: torch.Tensor, kv: KvState, embeds: tuple | None = None) -> torch.Tensor:
        """Logits [T, vocab] (fp32) for the new tokens appended to ``kv``."""
        return self.head(self.hidden_states(tokens, kv, embeds))

    def mtp_forward(self, j: int, h_prev: torch.Tensor, next_tokens: torch.Tensor, positions: torch.Tensor,
                    kv: KvState) -> tuple[torch.Tensor, torch.Tensor]:
        """MTP depth j: pair (h_t, embed(x_{t+1})) -> norms -> projection -> one decoder layer ->
        shared head, predicting x_{t+2} (python/reference/families/qwen4/mtp.py:1-32)."""
        cfg, p = self.cfg, self.p
        li = cfg.num_layers + j
        pre = f"model.layers.{li}."
        e = ops.rmsnorm(self.embed(next_tokens), p[pre + "enorm.weight"], cfg.rms_eps)
        hn = ops.rmsnorm(h_prev, p[pre + "hnorm.weight"], cfg.rms_eps)
        x = (torch.cat([e, hn], dim=-1).float() @ p[pre + "eh_proj.weight"].float().T).to(h_prev.dtype)
        h = self.layer(li, x, positions, kv)
        xn = ops.rmsnorm(h, p[pre + "shared_head.norm.weight"], cfg.rms_eps)
        w = p["model.embed_tokens.weight"] if cfg.tie_embeddings else p["lm_head.weight"]
        return xn.float() @ w.float().T, h

    @torch.no_grad()
    def generate(self, prompts: torch.Tensor, steps: int) -> tuple[torch.Tensor, torch.Tensor]:
        """Greedy decode.  prompts [B, T].  Returns (tokens [B, steps], logits [B, steps, vocab])."""
        B = prompts.shape[0]
        out_t, out_l = [], []
        for b in range(B):
            kv = KvState(self.cfg)
            logits = self.forward(prompts[b], kv)[-1:]
            toks, ls = [], []
            for _ in range(steps):
                ls.append(logits[0])
                t = logits.argmax(-1)
                toks.append(t)
                logits = self.forward(t, kv)
            out_t.append(torch.cat(toks))
            out_l.append(torch.stack(ls))
        return torch.stack(out_t), torch.stack(out_l)
