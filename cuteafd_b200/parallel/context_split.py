"""Context (token) split of attention over the ranks of a group: the KV of a sequence is partitioned by page parity
(logical page j lives on rank j mod n), heads are split for the projections, and one attention layer needs three
exchanges:

    1. query all-gather            every rank projects the queries of its own heads; [R, H/n, D] -> [R, H, D]
    2. partial attention           every rank attends, for ALL heads, over the pages it holds and produces an
                                   unnormalised output with its base-2 log-sum-exp state (m, l) per row and head
    3. partial + LSE exchange      the partials of a head go to the rank that owns the head, which merges them in
                                   rank order (fixed order: the same bits on every run) and continues with its
                                   slice of the output projection

With a sparse-attention indexer there is a fourth: every rank scores its own positions, keeps its local top-k, and the
candidate lists ([R, k] scores and positions per rank) are merged into the global top-k (ties to the lower
position) before step 2.

This module is the host-side form: plain tensor math per rank and ``torch.distributed`` collectives, which is what the
CPU oracle and the gloo tests run.  On GPUs the same three steps map onto kernels that already exist: the split-KV
attention kernels write exactly these partials (unnormalised O, m, l per split) and ``*_merge_kernel`` merges them in
split order, so a rank's partials become "splits" of the owner's merge; that binding is not wired yet.

Counterpart: rust/crates/cuteafd-daemon/src/shared/peer_split/context.rs:1-90 (degree 2, query all-gather, candidate
merge, partial + LSE combine) and native/shared/cuda/attention.cu:925 (state merge).
"""
from __future__ import annotations

import math

import torch
import torch.distributed as dist

PAGE = 64
LOG2E = 1.4426950408889634


def page_owner(position: torch.Tensor | int, ranks: int, page: int = PAGE):
    """Rank that holds a KV position: pages are dealt round-robin."""
    return (position // page) % ranks


def local_positions(kv_len: int, rank: int, ranks: int, page: int = PAGE) -> torch.Tensor:
    """Positions [0, kv_len) this rank holds, ascending."""
    pos = torch.arange(kv_len)
    return pos[page_owner(pos, ranks, page) == rank]


def partial_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, k_pos: torch.Tensor, q_pos: torch.Tensor,
                      scale: float, allowed: torch.Tensor | None = None):
    """Attention of q [R, H, D] over the local keys k [L, Hk, D] / values v [L, Hk, Dv] at positions ``k_pos`` [L];
    query row r sits at ``q_pos[r]`` and sees positions <= its own (and, with ``allowed`` [R, L], only those).
    Returns (o [R, H, Dv] unnormalised fp32, m [R, H] base-2 maximum, l [R, H] sum of 2^(s - m)); a row that sees
    nothing here has m = -inf, l = 0, o = 0."""
    R, H, _ = q.shape
    rep = H // k.shape[1]
    kf, vf = k.float().repeat_interleave(rep, dim=1), v.float().repeat_interleave(rep, dim=1)
    s = torch.einsum("rhd,lhd->rhl", q.float(), kf) * (scale * LOG2E)
    vis = k_pos[None, :] <= q_pos[:, None]
    if allowed is not None:
        vis = vis & allowed
    s = s.masked_fill(~vis[:, None, :], float("-inf"))
    m = s.max(dim=-1).values if s.shape[-1] else torch.full((R, H), float("-inf"))
    safe = torch.where(torch.isinf(m), torch.zeros_like(m), m)
    p = torch.exp2(s - safe[..., None])
    p = torch.where(vis[:, None, :], p, torch.zeros_like(p))
    return torch.einsum("rhl,lhd->rhd", p, vf), m, p.sum(dim=-1)


def merge_partials(parts: list) -> torch.Tensor:
    """[(o, m, l), ...] in rank order -> normalised output [R, H, Dv] (fp32).  Fixed order, base-2 states."""
    o, m, l = (t.clone() for t in parts[0])
    for o2, m2, l2 in parts[1:]:
        m_new = torch.maximum(m, m2)
        safe = torch.where(torch.isinf(m_new), torch.zeros_like(m_new), m_new)
        a = torch.where(torch.isinf(m), torch.zeros_like(m), torch.exp2(m - safe))
        b = torch.where(torch.isinf(m2), torch.zeros_like(m2), torch.exp2(m2 - safe))
        o = o * a[..., None] + o2 * b[..., None]
        l = l * a + l2 * b
        m = m_new
    return o / l.clamp_min(1e-30)[..., None]


def merge_candidates(scores: list, positions: list, top_k: int) -> torch.Tensor:
    """Per-rank candidate lists ([R, k_r] scores, [R, k_r] positions, -1 = empty slot) -> global top-k positions [R, top_k]
    ascending, -1 padded; higher score first, ties to the lower position."""
    s = torch.cat(scores, dim=1).float()
    p = torch.cat(positions, dim=1).long()
    s = torch.where(p < 0, torch.full_like(s, float("-inf")), s)
    R = s.shape[0]
    out = torch.full((R, top_k), -1, dtype=torch.long)
    for r in range(R):
        valid = p[r] >= 0
        ps, ss = p[r][valid], s[r][valid]
        order = sorted(range(ps.numel()), key=lambda i: (-float(ss[i]), int(ps[i])))[:top_k]
        chosen = torch.sort(ps[order]).values
        out[r, :chosen.numel()] = chosen
    return out


class ContextSplit:
    """One rank's view.  ``heads`` are split contiguously: rank r owns heads [r * H/n, (r + 1) * H/n)."""

    def __init__(self, group=None, page: int = PAGE):
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.page = page

    def gather_queries(self, q_own: torch.Tensor) -> torch.Tensor:
        """[R, H/n, D] of this rank's heads -> [R, H, D]."""
        parts = [torch.empty_like(q_own) for _ in range(self.ranks)]
        dist.all_gather(parts, q_own.contiguous(), group=self.group)
        return torch.cat(parts, dim=1)

    def exchange_candidates(self, scores: torch.Tensor, positions: torch.Tensor, top_k: int) -> torch.Tensor:
        ss = [torch.empty_like(scores) for _ in range(self.ranks)]
        ps = [torch.empty_like(positions) for _ in range(self.ranks)]
        dist.all_gather(ss, scores.contiguous(), group=self.group)
        dist.all_gather(ps, positions.contiguous(), group=self.group)
        return merge_candidates(ss, ps, top_k)

    def attend(self, q_own: torch.Tensor, k_local: torch.Tensor, v_local: torch.Tensor, k_pos: torch.Tensor, q_pos: torch.Tensor,
               scale: float | None = None, allowed: torch.Tensor | None = None) -> torch.Tensor:
        """Whole step for this rank: returns the normalised attention output of its own heads [R, H/n, Dv] (fp32)."""
        q = self.gather_queries(q_own)
        scale = scale if scale is not None else 1.0 / math.sqrt(q.shape[-1])
        o, m, l = partial_attention(q, k_local, v_local, k_pos, q_pos, scale, allowed)
        # every rank needs every rank's partial of ITS heads: gather the packed (o | m | l) states and keep the slice
        packed = torch.cat([o, m[..., None], l[..., None]], dim=-1).contiguous()
        every = [torch.empty_like(packed) for _ in range(self.ranks)]
        dist.all_gather(every, packed, group=self.group)
        hn = q_own.shape[1]
        lo = self.rank * hn
        dv = o.shape[-1]
        parts = [(e[:, lo:lo + hn, :dv], e[:, lo:lo + hn, dv], e[:, lo:lo + hn, dv + 1]) for e in every]
        return merge_partials(parts)
