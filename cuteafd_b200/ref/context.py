"""The oracle decoder with its attention context-split over the ranks of a group (GQA families).

Every rank holds all weights and runs the whole residual stream (that part of the reference's TP2 is covered by the
head-split engine); what is split here is what the context split splits: a rank keeps K / V only for the pages it owns
(logical page j on rank j mod n), projects the queries of its own heads, and attention runs as the three exchanges of
``parallel/context_split.py`` — query all-gather, partial attention with log-sum-exp states over the local pages,
partial exchange and fixed-order merge at the head's owner — followed by an all-gather of the heads' outputs for the
output projection.  Prefill and decode use the same path; a decode step's new K / V row lands on whichever rank owns
its page.

The logits must equal the whole decoder's up to fp32 summation order (the merge adds the ranks' partial sums in rank
order instead of one pass over the keys), which is what the gloo test checks over a prompt and several decode steps.

Counterpart: rust/crates/cuteafd-daemon/src/shared/peer_split/context.rs:1-90 inside the family engines' layer loop.
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..parallel import context_split as CS
from . import ops
from .model import KvState, RefDecoder


class ContextKv(KvState):
    """One rank's share of a sequence's KV: the rows of the pages it owns, their positions, and the sequence's whole
    length (which is what the next step's positions follow from)."""

    def __init__(self, cfg: ModelConfig):
        super().__init__(cfg)
        self.total = 0
        self.local_pos: dict[int, torch.Tensor] = {}

    def length(self, layer: int = 0) -> int:
        return self.total

    def held(self, layer: int = 0) -> int:
        return super().length(layer)


class ContextSplitDecoder(RefDecoder):
    def __init__(self, cfg: ModelConfig, params: dict[str, torch.Tensor], group=None):
        if cfg.is_mla:
            raise ValueError("the context-split oracle covers the GQA families")
        super().__init__(cfg, params)
        self.cs = CS.ContextSplit(group)
        if cfg.num_heads % self.cs.ranks or cfg.num_kv_heads % 1:
            raise ValueError("heads must divide over the ranks")

    def attention(self, layer: int, x: torch.Tensor, positions: torch.Tensor, kv: KvState) -> torch.Tensor:
        cfg, p, cs = self.cfg, self.p, self.cs
        a = f"model.layers.{layer}.self_attn."
        T = x.shape[0]
        hn = cfg.num_heads // cs.ranks
        lo = cs.rank * hn
        # queries of this rank's heads only; keys / values of every head, kept only for the pages this rank owns
        wq = p[a + "q_proj.weight"].float().view(cfg.num_heads, cfg.head_dim, -1)[lo:lo + hn].reshape(hn * cfg.head_dim, -1)
        q = (x.float() @ wq.T).to(x.dtype).view(T, hn, cfg.head_dim)
        k = (x.float() @ p[a + "k_proj.weight"].float().T).to(x.dtype).view(T, cfg.num_kv_heads, cfg.head_dim)
        v = (x.float() @ p[a + "v_proj.weight"].float().T).to(x.dtype).view(T, cfg.num_kv_heads, cfg.head_dim)
        if cfg.qk_norm:
            q = ops.rmsnorm(q, p[a + "q_norm.weight"], cfg.rms_eps)
            k = ops.rmsnorm(k, p[a + "k_norm.weight"], cfg.rms_eps)
        q = ops.apply_rope(q, positions, cfg.rope_theta, cfg.rope_interleaved, self.inv_freq, self.rope_mag)
        k = ops.apply_rope(k, positions, cfg.rope_theta, cfg.rope_interleaved, self.inv_freq, self.rope_mag)
        mine = CS.page_owner(positions, cs.ranks) == cs.rank
        rec = torch.cat([k.reshape(T, -1), v.reshape(T, -1)], dim=-1)[mine]
        full = kv.append(layer, rec)                           # this rank's rows only
        prev = kv.local_pos.get(layer, positions.new_empty(0))
        kv.local_pos[layer] = torch.cat([prev, positions[mine]])
        if layer == 0:
            kv.total = int(positions[-1]) + 1                  # positions of this step were fixed before the layer loop
        half = cfg.num_kv_heads * cfg.head_dim
        k_loc = full[:, :half].view(-1, cfg.num_kv_heads, cfg.head_dim)
        v_loc = full[:, half:].view(-1, cfg.num_kv_heads, cfg.head_dim)
        o_own = cs.attend(q, k_loc, v_loc, kv.local_pos[layer], positions, self.scale_mul / math.sqrt(cfg.head_dim))
        o_own = o_own.to(x.dtype)                              # the whole decoder rounds the attention output once, here
        parts = [torch.empty_like(o_own) for _ in range(cs.ranks)]
        dist.all_gather(parts, o_own.contiguous(), group=cs.group)
        o = torch.cat(parts, dim=1).reshape(T, cfg.num_heads * cfg.head_dim)
        return (o.float() @ p[a + "o_proj.weight"].float().T).to(x.dtype)

    def new_kv(self) -> ContextKv:
        return ContextKv(self.cfg)
