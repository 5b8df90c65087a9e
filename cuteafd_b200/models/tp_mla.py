"""Tensor-parallel attention ranks for the MLA family: heads split over the TP group, rows of the residual stream
sharded, the same fused collectives as the GQA form (models/tp_gqa.py).

Per layer, on every rank r of n:

    a       = x_full @ Wqkv_a.T            q_a / kv_a (+ rope key) of every row on every rank: the latent cache is shared by
                                           all heads, so it is replicated and every rank writes every record
                                                                                                  [all-gather -> GEMM]
    q_r     = q_a @ Wq_b_r.T               this rank's heads; absorbed through its W_uk heads
    attn_r  = MLA attention(local heads)   over the replicated latent pages, un-absorbed through its W_uv heads
    partial = attn_r @ Wo_r.T              row-parallel, epilogue stores every row at its owner  [GEMM -> reduce-scatter]
    h_own  += sum_r partial ; x = norm2(h)                                                       [reduce + norm + all-gather]

and the FFN half runs on the owned rows as in the GQA engine.  The reference splits the MLA heads of its large
checkpoints over two coordinator GPUs (rust/crates/cuteafd-loader/src/placement/mod.rs:303-311; "2 RTX (head split)"
layouts of its release cards).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import ModelConfig
from .mla_moe import LatentCache, MlaLayerWeights, MlaMoeEngine, MlaMoeWeights
from .gqa_moe import LayerWeights
from .tp_gqa import TpGqaMoeEngine


def shard_mla_weights(cfg: ModelConfig, W: MlaMoeWeights, rank: int, ranks: int) -> MlaMoeWeights:
    """The weights rank ``rank`` serves: q_b rows, W_uk / W_uv / k_b heads and o columns of its heads; q_a / kv_a, norms and
    the FFN half shared.  The E4M3 twins of the whole projections are dropped (decode-sized steps take the bf16 shards)."""
    assert cfg.num_heads % ranks == 0
    hl = cfg.num_heads // ranks
    h0, h1 = rank * hl, (rank + 1) * hl
    qd, vd, nd = cfg.qk_head_dim, cfg.v_head_dim, cfg.qk_nope_dim
    out = MlaMoeWeights.__new__(MlaMoeWeights)
    out.__dict__.update(W.__dict__)
    out.layers = []
    for L in W.layers:
        S = MlaLayerWeights()
        for name in LayerWeights.__slots__ + MlaLayerWeights.__slots__:
            setattr(S, name, getattr(L, name))
        S.wq_b = L.wq_b[h0 * qd:h1 * qd].contiguous()
        S.w_uk, S.w_uv = L.w_uk[h0:h1].contiguous(), L.w_uv[h0:h1].contiguous()
        S.w_kb = L.w_kb[h0 * nd:h1 * nd].contiguous() if L.w_kb is not None else None
        S.wo = L.wo[:, h0 * vd:h1 * vd].contiguous()
        S.fp8 = None
        out.layers.append(S)
    return out


class TpMlaMoeEngine(TpGqaMoeEngine, MlaMoeEngine):
    """One rank of a tensor-parallel MLA attention group.  Every rank is given the same batches; ``forward`` (the GQA
    form's: embedding of the owned rows, per-layer attention + owned-row FFN, sharded or whole head) returns the same
    logits on every rank.  Dense MLA only: the lightning indexer's scores are not split."""

    def __init__(self, cfg: ModelConfig, weights: MlaMoeWeights, num_pages: int, max_tokens: int, max_seqs: int = 64,
                 group=None, build_moe: bool = True, shard_head: bool = False):
        if cfg.indexer_heads:
            raise ValueError("tensor-parallel MLA serves dense attention (no lightning indexer)")
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.full_cfg = cfg
        local = cfg.replace(num_heads=cfg.num_heads // self.ranks, mtp_layers=0)
        dev = weights.embed.device
        sharded = shard_mla_weights(cfg, weights, self.rank, self.ranks)
        MlaMoeEngine.__init__(self, local, sharded, LatentCache(local, num_pages, dev), max_tokens, max_seqs, build_moe=build_moe)
        self._init_tp(cfg, weights, max_tokens, max_seqs, shard_head)

    _attention = MlaMoeEngine._attention

    def _x_rows(self, T: int) -> torch.Tensor:
        return self.tp.x_full[:T]

    def _proj_a(self, L, T: int) -> None:
        self.tp.column_parallel_linear(T, L.wqkv_a, self.ws.a[:T])

    def _proj_o(self, L, T: int, twin: bool = True) -> None:
        tp = self.tp
        tp.step()
        tp.row_parallel_linear(self.ws.attn[:T], L.wo)
        tp.reduce_norm_gather(T, L.ln2, self.cfg.rms_eps)
        self.collectives += 2
