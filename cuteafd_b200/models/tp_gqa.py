"""Tensor-parallel attention ranks for the GQA MoE family: heads split over the TP group, rows of the residual
stream sharded, collectives fused into the kernels.

Per layer, on every rank r of n (R = ceil(T / n) rows owned):

    qkv_r   = x_full @ Wqkv_r.T            column-parallel GEMM over the gathered activations; the kernel waits for the
                                           gather flags itself                                   [all-gather -> GEMM]
    attn_r  = attention(local heads)       local q heads, local kv heads, local pages of the KV cache
    partial = attn_r @ Wo_r.T              row-parallel GEMM, epilogue stores every row at its owner over NVLink
                                                                                                  [GEMM -> reduce-scatter]
    h_own  += sum_r partial ; x = norm2(h) owner adds in rank order, normalises, pushes x rows to every rank
                                                                                                  [reduce + norm + all-gather]
    y_own   = FFN(x_own)                   the FFN half is data-parallel over the owned rows: router, dispatch, experts,
                                           combine (a local exchange here; the AFD exchange takes the same rows)
    h_own  += y_own ; x = norm1'(h)        next layer's input norm, pushed to every rank          [norm + all-gather]

so a layer costs one reduce-scatter and two all-gathers of activations, all of them inside kernels that also do
the neighbouring math, and no rank computes a row of the FFN that another rank owns.

The reference splits heads over two coordinator GPUs with a replicated residual and a push / wait / ordered-add
all-reduce (rust/crates/cuteafd-loader/src/placement/mod.rs:303-311, rust/crates/cuteafd-daemon/src/shared/
peer_split/attention.rs, native/shared/cuda/peer_exchange.cu:259-263); this engine keeps its fixed-order fp32 sum and
shards the rows instead, for any degree that divides the kv heads.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..ops import kernels as K
from ..parallel.tp import TpContext
from .gqa_moe import Batch, GqaMoeEngine, GqaMoeWeights, KvCache, LayerWeights


def shard_attention_weights(cfg: ModelConfig, W: GqaMoeWeights, rank: int, ranks: int) -> GqaMoeWeights:
    """The weights rank ``rank`` serves: q / k / v rows and o columns of its heads; everything else shared."""
    assert cfg.num_kv_heads % ranks == 0 and cfg.num_heads % ranks == 0
    D, hq, hk = cfg.head_dim, cfg.num_heads // ranks, cfg.num_kv_heads // ranks
    q0, k0, v0 = 0, cfg.num_heads * D, (cfg.num_heads + cfg.num_kv_heads) * D
    out = GqaMoeWeights.__new__(GqaMoeWeights)
    out.__dict__.update(W.__dict__)
    out.layers = []
    for L in W.layers:
        S = LayerWeights()
        for name in LayerWeights.__slots__:
            setattr(S, name, getattr(L, name))
        S.wqkv = torch.cat([L.wqkv[q0 + rank * hq * D: q0 + (rank + 1) * hq * D],
                            L.wqkv[k0 + rank * hk * D: k0 + (rank + 1) * hk * D],
                            L.wqkv[v0 + rank * hk * D: v0 + (rank + 1) * hk * D]]).contiguous()
        if L.bqkv is not None:
            S.bqkv = torch.cat([L.bqkv[q0 + rank * hq * D: q0 + (rank + 1) * hq * D],
                                L.bqkv[k0 + rank * hk * D: k0 + (rank + 1) * hk * D],
                                L.bqkv[v0 + rank * hk * D: v0 + (rank + 1) * hk * D]]).contiguous()
        S.wo = L.wo[:, rank * hq * D:(rank + 1) * hq * D].contiguous()
        out.layers.append(S)
    return out


class TpGqaMoeEngine(GqaMoeEngine):
    """One rank of a tensor-parallel attention group.  Every rank is given the same batches; ``forward`` returns the
    same logits on every rank."""

    def __init__(self, cfg: ModelConfig, weights: GqaMoeWeights, num_pages: int, max_tokens: int, max_seqs: int = 64,
                 group=None, build_moe: bool = True, shard_head: bool = False):
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.full_cfg = cfg
        local = cfg.replace(num_heads=cfg.num_heads // self.ranks, num_kv_heads=cfg.num_kv_heads // self.ranks)
        dev = weights.embed.device
        sharded = shard_attention_weights(cfg, weights, self.rank, self.ranks)
        super().__init__(local, sharded, KvCache(local, num_pages, dev), max_tokens, max_seqs, build_moe=build_moe)
        self._init_tp(cfg, weights, max_tokens, max_seqs, shard_head)

    def _init_tp(self, cfg: ModelConfig, weights, max_tokens: int, max_seqs: int, shard_head: bool) -> None:
        """The tensor-parallel half of the construction: symmetric buffers, owned-row output, the sharded head."""
        dev = self.device
        self.tp = TpContext(cfg.hidden, max_tokens, dev, self.group)
        self.own_out = torch.zeros(self.tp.max_rows_per_rank, cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.collectives = 0
        # Vocabulary-sharded head: this rank keeps rows [lo, hi) of the head only, ``forward`` returns its slice of the
        # logits, ``greedy`` exchanges per-rank winners (8 bytes per row and rank) and ``full_logits`` gathers the slices
        # for rows that are sampled (rust/crates/cuteafd-daemon/src/shared/distributed_head.rs).
        self.shard_head = shard_head
        if shard_head:
            from ..parallel.head import shard_rows
            self.head_lo, self.head_hi = shard_rows(cfg.vocab_size, self.ranks, self.rank)
            self.head_per = shard_rows(cfg.vocab_size, self.ranks, 0)[1]
            self.head_w = weights.lm_head[self.head_lo:self.head_hi].contiguous()
            self.W.lm_head = None                                        # the full head is not kept on this rank
            self.logits = None
            self.local_logits = torch.zeros(max_seqs, max(self.head_per, 1), dtype=torch.float32, device=dev)

    def collect_max(self, ms: float) -> float:
        """Largest device time over the ranks of the group (benchmarks report the slowest rank)."""
        t = torch.tensor([ms], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX, group=self.group)
        return float(t.item())

    # owned rows of the current step
    def _own(self, T: int) -> tuple[int, int]:
        lo = self.rank * self.tp.rows_per_rank
        return lo, self.tp.rows_owned(T)

    def _attention(self, i: int, T: int, b: Batch) -> None:
        cfg, L, ws, tp = self.cfg, self.W.layers[i], self.ws, self.tp
        tp.column_parallel_linear(T, L.wqkv, ws.qkv[:T])
        K.qk_rope_kv(ws.qkv[:T], L.q_norm, L.k_norm, self.inv_freq, b.positions, b.slots, ws.q[:T], self.kv.k[i],
                     self.kv.v[i], cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.rms_eps, cfg.rope_interleaved, bias=L.bqkv)
        if b.prefill:
            K.attn_prefill(ws.q[:T], self.kv.k[i], self.kv.v[i], b.page_table, b.seq_lens, b.q_start, ws.attn[:T], b.max_q_len,
                           window=cfg.window_of(i))
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
        tp.step()
        tp.row_parallel_linear(ws.attn[:T].view(T, -1), L.wo)
        tp.reduce_norm_gather(T, L.ln2, cfg.rms_eps)
        self.launches += 6
        self.collectives += 2

    def _ffn_own(self, i: int, T: int) -> torch.Tensor | None:
        """FFN of the owned rows (their normalised input sits in this rank's copy of ``x_full``); returns the rows to
        add to the residual, or None when this rank owns no row of the step."""
        cfg, L, ws, tp = self.cfg, self.W.layers[i], self.ws, self.tp
        lo, n = self._own(T)
        if n == 0:
            return None
        x = tp.x_full[lo:lo + n]
        y = self.own_out[:n]
        if L.router is None:
            K.linear(x, L.d_gate, out=ws.ffn_d[:n], w_up=L.d_up)
            K.linear(ws.ffn_d[:n], L.d_down, out=y)
            self.launches += 2
            return y
        logits = K.linear(x, L.router, out=ws.router[:n, :cfg.num_experts], out_f32=True)
        shared = None
        if L.s_gate is not None:
            K.linear(x, L.s_gate, out=ws.ffn_s[:n], w_up=L.s_up)
            shared = K.linear(ws.ffn_s[:n], L.s_down, out=ws.shared[:n])
            self.launches += 2
        if self.pre_moe is not None:
            self.pre_moe(i)
        self.moe.forward(x, logits, dict(self.route_kw, bias=L.router_bias), L.w_gate, L.w_up, L.w_down, y, shared=shared)
        self.launches += 6
        return y

    def forward(self, b: Batch) -> torch.Tensor:
        cfg, ws, tp = self.cfg, self.ws, self.tp
        T = b.tokens.shape[0]
        assert T <= self.max_tokens
        tp.set_rows(T)
        lo, n = self._own(T)
        if n:
            K.embed(b.tokens[lo:lo + n], self.W.embed, out=tp.residual[:n])
        tp.wait_buffers_free()           # the peers have read what the previous step gathered here
        tp.step()
        tp.reduce_norm_gather(T, self.W.layers[0].ln1, cfg.rms_eps, gather_only=True)
        self.launches += 2
        self.collectives += 1
        for i in range(cfg.num_layers):
            self._attention(i, T, b)
            y = self._ffn_own(i, T)
            nxt = self.W.layers[i + 1].ln1 if i + 1 < cfg.num_layers else self.W.final_norm
            tp.step()
            if y is None:
                tp.reduce_norm_gather(T, nxt, cfg.rms_eps, gather_only=True)
            else:
                tp.reduce_norm_gather(T, nxt, cfg.rms_eps, local=y)
            self.launches += 1
            self.collectives += 1
        # x_full now holds final_norm(h) of every row on every rank
        tp.wait_gathered()
        rows = tp.x_full[:T].index_select(0, b.last_rows) if b.last_rows is not None else tp.x_full[:T]
        n_out = rows.shape[0]
        if self.shard_head:
            if n_out > self.local_logits.shape[0]:
                self.local_logits = torch.zeros(n_out, self.local_logits.shape[1], dtype=torch.float32, device=self.device)
            logits = self.local_logits[:n_out, :self.head_hi - self.head_lo]
            if self.head_hi > self.head_lo:
                K.linear(rows.contiguous(), self.head_w, out=logits, out_f32=True)
        else:
            logits = K.linear(rows.contiguous(), self.W.lm_head, out=self.logits[:n_out], out_f32=True)
        tp.release_buffers()
        self.launches += 3 + 2 * self.ranks
        return logits

    def greedy(self, logits: torch.Tensor) -> torch.Tensor:
        if not self.shard_head:
            return super().greedy(logits)
        self.launches += 2
        self.collectives += 1
        return self.tp.head_pick(logits, self.head_lo, self.next_tokens[:logits.shape[0]])

    def full_logits(self, logits: torch.Tensor) -> torch.Tensor:
        """Whole-vocabulary logits [T, vocab] on every rank from the slices (rows that are sampled, not argmax'ed)."""
        if not self.shard_head:
            return logits
        T = logits.shape[0]
        pad = torch.full((T, self.head_per), float("-inf"), dtype=torch.float32, device=self.device)
        pad[:, :logits.shape[1]] = logits
        parts = torch.empty(self.ranks, T, self.head_per, dtype=torch.float32, device=self.device)
        dist.all_gather_into_tensor(parts.view(-1), pad.view(-1), group=self.group)
        return parts.permute(1, 0, 2).reshape(T, -1)[:, :self.full_cfg.vocab_size]
