"""Vocabulary-sharded LM head: every attention rank holds a contiguous slice of the head's rows, computes its
slice of the logits with the tcgen05 GEMM, reduces it to per-row candidates on the device, and only the candidates
cross the fabric.

Greedy rows exchange (best value, best id) per rank: 8 bytes per row and rank instead of a vocabulary-wide logit
row; the global winner is the highest value with ties to the lowest id, which is exactly the single-GPU argmax
rule.  Sampled rows need the whole distribution; ``gather_logits`` assembles it (slice by slice) for the exact
sampler.  Reference: the distributed head of the coordinator pair
(rust/crates/cuteafd-daemon/src/shared/distributed_head.rs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist


def shard_rows(vocab: int, ranks: int, rank: int, multiple: int = 128) -> tuple[int, int]:
    """Row range of ``rank``: equal shares rounded up to ``multiple`` rows (the GEMM's feature tile)."""
    per = -(-vocab // ranks)
    per = -(-per // multiple) * multiple
    lo = min(vocab, rank * per)
    return lo, min(vocab, lo + per)


class ShardedHead:
    def __init__(self, head_shard: torch.Tensor, vocab: int, group=None, linear=None, argmax=None):
        """``head_shard`` = rows [lo, hi) of the head [vocab, H].  ``linear`` / ``argmax`` default to the CUDA
        kernels; CPU tests pass torch functions."""
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.vocab = vocab
        self.lo, self.hi = shard_rows(vocab, self.ranks, self.rank)
        assert head_shard.shape[0] == self.hi - self.lo
        self.w = head_shard
        if linear is None:
            from ..ops import kernels as K
            linear = lambda x, w: K.linear(x, w, out_f32=True)                                  # noqa: E731
            argmax = lambda lg: K.argmax(lg).long()                                             # noqa: E731
        self.linear, self.argmax = linear, argmax

    def local_logits(self, x: torch.Tensor) -> torch.Tensor:
        return self.linear(x, self.w)

    def greedy(self, x: torch.Tensor) -> torch.Tensor:
        """Global argmax ids [T] (identical on every rank)."""
        lg = self.local_logits(x)
        T = lg.shape[0]
        if lg.shape[1] == 0:
            best_v = torch.full((T,), float("-inf"), device=x.device)
            best_i = torch.zeros(T, dtype=torch.long, device=x.device)
        else:
            best_i = self.argmax(lg)
            best_v = lg.gather(1, best_i[:, None])[:, 0]
            best_v = torch.where(torch.isnan(best_v), torch.full_like(best_v, float("-inf")), best_v)
        cand = torch.stack([best_v.float(), (best_i + self.lo).float()], 1).contiguous()          # ids < 2^24: exact in fp32
        allc = [torch.empty_like(cand) for _ in range(self.ranks)]
        dist.all_gather(allc, cand, group=self.group)
        vals = torch.stack([c[:, 0] for c in allc], 1)                                              # [T, ranks], rank order = id order
        ids = torch.stack([c[:, 1] for c in allc], 1)
        top = vals.max(1, keepdim=True).values
        first = (vals == top).float().argmax(1)                                                     # lowest rank among ties = lowest id
        return ids.gather(1, first[:, None])[:, 0].long()

    def gather_logits(self, x: torch.Tensor) -> torch.Tensor:
        """Full logits [T, vocab] on every rank (for rows that are sampled, not argmax'ed)."""
        lg = self.local_logits(x).float()
        per = shard_rows(self.vocab, self.ranks, 0)[1]
        pad = torch.full((lg.shape[0], per), float("-inf"), device=lg.device)
        pad[:, :lg.shape[1]] = lg
        parts = [torch.empty_like(pad) for _ in range(self.ranks)]
        dist.all_gather(parts, pad, group=self.group)
        return torch.cat(parts, 1)[:, :self.vocab]
