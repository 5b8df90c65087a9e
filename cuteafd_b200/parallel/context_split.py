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

The first half of this module is the host-side form: plain tensor math per rank and ``torch.distributed`` collectives,
which is what the CPU oracle and the gloo tests run.  The second half (``DeviceContextSplit``, ``ContextSplitEngine``,
``ContextSplitDriver``) is the GPU form for the GQA family: the split-KV decode attention kernel runs over the pages a
rank holds and stores its partials (unnormalised O, m, l per split) straight into every rank's scratch over NVLink, a
flag per peer publishes them, and the merge kernel walks all ranks' partials in rank order, so a rank's partials are
simply further "splits" of one merge.  Step 1 costs nothing there because every rank projects all heads (the
projections are replicated; what the split buys is KV capacity and attention bandwidth for long contexts).

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


# ---- GPU form --------------------------------------------------------------------------------------------------------
class DeviceContextSplit:
    """Symmetric scratch + flags of a context-split group.  ``attend`` = partial attention over the local pages (stored
    into every rank's scratch) -> publish -> wait for every rank -> merge.  Two scratch buffers alternate, so a fast
    rank's partials of the next layer never land in a buffer a slow rank is still merging (it cannot run two layers
    ahead: its own merge of the next layer waits for the slow rank's partials)."""

    def __init__(self, num_heads: int, num_kv_heads: int, head_dim: int, max_seqs: int, max_q_len: int, splits: int,
                 device: torch.device, group=None, mla: bool = False):
        from ..ops import kernels as K
        from .afd import SymmetricHeap, _align
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.Hq, self.Hkv, self.D, self.splits, self.device = num_heads, num_kv_heads, head_dim, splits, device
        self.max_seqs, self.max_q_len = max_seqs, max_q_len
        if mla:        # absorbed MLA: row blocks of 128 (token, head) pairs, two output halves each
            self.max_blocks = max_seqs * ((max_q_len * num_heads + 127) // 128)
            floats = K.mla_scratch_floats(self.max_blocks, splits * self.ranks)
        else:
            floats = K.attn_decode_scratch_floats(max_seqs, max_q_len, num_heads, num_kv_heads, splits * self.ranks)
        self.buf_bytes = _align(floats * 4)
        self.off_flags = 2 * self.buf_bytes
        self.heap = SymmetricHeap(self.off_flags + 1024, device, self.group)
        self.scratch = [self.heap.view(i * self.buf_bytes, floats * 4, torch.float32) for i in range(2)]
        self.flags = self.heap.view(self.off_flags, 64, torch.int32)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.turn = 0
        import ctypes as C
        self._flag_ptrs = (C.c_void_p * 8)(*[self.heap.ptrs[r] + self.off_flags + 4 * self.rank for r in range(self.ranks)])

    def _exchange(self, partial, merge):
        """``partial(peer scratch addresses)`` stores this rank's partials everywhere; ``merge(own scratch)`` runs once
        every rank's flag of this turn has arrived."""
        from .._native import lib as _n
        from ..ops import kernels as K
        b = self.turn & 1
        self.turn += 1
        K.bump_epoch(self.epoch)
        partial([self.heap.ptrs[r] + b * self.buf_bytes for r in range(self.ranks)])
        _n.check(_n.cuda_lib().cafd_tp_signal(self._flag_ptrs, self.ranks, self.epoch.data_ptr(), K._stream()), "context split signal")
        for r in range(self.ranks):
            K.wait_flag(self.flags.data_ptr() + 4 * r, self.epoch)
        return merge(self.scratch[b])

    def attend(self, q, k_cache, v_cache, page_table, seq_lens, kv_base, q_start, out, max_q_len: int):
        """q [T, Hq, D] (all heads), local page table / local lengths / visibility bases -> out [T, Hq, D] on every rank."""
        from ..ops import kernels as K
        assert page_table.shape[0] <= self.max_seqs and max_q_len <= self.max_q_len
        return self._exchange(
            lambda peers: K.attn_decode_partial(q, k_cache, v_cache, page_table, seq_lens, kv_base, q_start, peers, self.rank,
                                                max_q_len, self.splits),
            lambda mine: K.attn_merge(mine, q_start, out, max_q_len, self.Hkv, self.splits * self.ranks))

    def attend_mla(self, q_abs, cache, page_table, seq_lens, kv_base, q_start, block_seq, block_tok0, out, scale: float, out_tpad: int):
        """Absorbed MLA: q_abs [T, heads, 576] (all heads), this rank's latent records -> out head-major
        [heads, out_tpad, 512] on every rank."""
        from ..ops import kernels as K
        assert block_seq.numel() <= self.max_blocks
        return self._exchange(
            lambda peers: K.mla_attention_partial(q_abs, cache, page_table, seq_lens, kv_base, q_start, block_seq, block_tok0, peers,
                                                  self.rank, scale, self.splits),
            lambda mine: K.mla_merge(mine, block_seq, block_tok0, q_start, out, self.Hq, self.splits * self.ranks, out_tpad))


def local_pages(n_pages: int, rank: int, ranks: int) -> int:
    """How many of the logical pages [0, n_pages) rank ``rank`` holds."""
    return max(0, (n_pages - rank + ranks - 1) // ranks)


def local_len(kv_len: int, rank: int, ranks: int, page: int = PAGE) -> int:
    """How many of the positions [0, kv_len) rank ``rank`` holds."""
    full, tail = divmod(kv_len, page)
    n = local_pages(full, rank, ranks) * page
    return n + (tail if full % ranks == rank else 0)


def make_engine(cfg, weights, num_pages: int, max_tokens: int, max_seqs: int, group=None, splits: int = 4):
    """An engine whose attention reads a context-split KV cache (GQA K / V pages, or MLA latent records in the absorbed
    form).  Everything else is the single-GPU engine, replicated on every rank of the group."""
    from ..models.gqa_moe import GqaMoeEngine, KvCache
    from ..ops import kernels as K
    if cfg.sliding_window:
        raise ValueError("context split and sliding-window layers do not combine: a window never spans more pages than one rank holds")
    if cfg.is_mla:
        from ..models.mla_moe import LatentCache, MlaMoeEngine
        if cfg.indexer_heads or cfg.kv_format != "bf16":
            raise ValueError("context split serves dense MLA over bf16 records (a sparse selection names global positions)")
        dev = weights.embed.device
        eng = MlaMoeEngine(cfg, weights, LatentCache(cfg, num_pages, dev), max_tokens, max_seqs)
        # (slots are -1 on the ranks that do not hold the page of a new token: mla_prep_a drops the record there)
        eng.cs = eng.kv_exchange = DeviceContextSplit(cfg.num_heads, 1, 576, max_seqs, PAGE, splits, dev, group, mla=True)
        return eng

    class ContextSplitEngine(GqaMoeEngine):
        def __init__(self):
            dev = weights.embed.device
            super().__init__(cfg, weights, KvCache(cfg, num_pages, dev), max_tokens, max_seqs)
            self.cs = DeviceContextSplit(cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, max_seqs, PAGE, splits, dev, group)

        def _attention(self, i: int, T: int, b) -> None:
            c, L, ws = self.cfg, self.W.layers[i], self.ws
            K.linear(ws.x[:T], L.wqkv, out=ws.qkv[:T])
            # slots are -1 on the ranks that do not hold the page of a new token: their K / V rows are dropped there
            K.qk_rope_kv(ws.qkv[:T], L.q_norm, L.k_norm, self.inv_freq, b.positions, b.slots, ws.q[:T], self.kv.k[i],
                         self.kv.v[i], c.num_heads, c.num_kv_heads, c.head_dim, c.rms_eps, c.rope_interleaved, bias=L.bqkv)
            self.cs.attend(ws.q[:T], self.kv.k[i], self.kv.v[i], b.page_table, b.seq_lens, b.kv_base, b.q_start, ws.attn[:T],
                           b.max_q_len)
            K.linear(ws.attn[:T].view(T, -1), L.wo, out=ws.h[:T], residual=ws.h[:T])
            self.launches += 7 + self.cs.ranks

    return ContextSplitEngine()


class ContextSplitDriver:
    """Per-rank bookkeeping of a context-split cache: which physical pages hold this rank's share of every sequence,
    and the step descriptions (local page table, local lengths, visibility bases, KV slots) the engine wants.  Steps
    never span a page boundary (a prompt goes in page-sized chunks), so the new tokens of a step live on one rank."""

    def __init__(self, engine, num_pages: int, max_pages_per_seq: int):
        from ..runtime.native import make_pool
        self.eng, self.pool, self.max_pages = engine, make_pool(num_pages), max_pages_per_seq
        self.ranks, self.rank = engine.cs.ranks, engine.cs.rank
        self.pages: dict[int, list[int]] = {}
        self.kv_len: dict[int, int] = {}
        self._next = 0

    def new(self) -> int:
        s, self._next = self._next, self._next + 1
        self.pages[s], self.kv_len[s] = [], 0
        return s

    def free(self, s: int) -> None:
        for p in self.pages.pop(s):
            self.pool.release(p)
        del self.kv_len[s]

    def _batch(self, items: list[tuple[int, list[int]]]):
        """items: (sequence, new tokens) with every run inside one page."""
        from ..models.gqa_moe import Batch
        dev = self.eng.device
        S = len(items)
        toks, pos, slots, lens, base, qs = [], [], [], [], [], [0]
        table = torch.zeros(S, self.max_pages, dtype=torch.int32)
        for i, (s, new) in enumerate(items):
            start, n = self.kv_len[s], len(new)
            assert n and start // PAGE == (start + n - 1) // PAGE, "a step stays inside one page"
            owner = (start // PAGE) % self.ranks
            need = local_pages((start + n + PAGE - 1) // PAGE, self.rank, self.ranks)
            while len(self.pages[s]) < need:
                self.pages[s].append(self.pool.alloc())
            table[i, :len(self.pages[s])] = torch.tensor(self.pages[s], dtype=torch.int32)
            mine = owner == self.rank
            ll = local_len(start + n, self.rank, self.ranks)
            for j in range(n):
                p = start + j
                toks.append(new[j]); pos.append(p)
                slots.append(self.pages[s][(p // PAGE) // self.ranks] * PAGE + p % PAGE if mine else -1)
            lens.append(ll)
            base.append(ll - n if mine else ll)          # a rank without the new tokens: all it holds is in their past
            qs.append(qs[-1] + n)
            self.kv_len[s] = start + n
        t = lambda v: torch.tensor(v, dtype=torch.int32, device=dev)                    # noqa: E731
        b = Batch(t(toks), t(pos), t(slots), table.to(dev), t(lens), t(qs), max(len(n) for _, n in items), False,
                  t([q - 1 for q in qs[1:]]))
        b.kv_base = t(base)
        return b

    def prefill(self, s: int, tokens: list[int]) -> torch.Tensor:
        """Append a prompt in page-sized chunks; returns the logits after its last token [1, vocab]."""
        logits, i = None, 0
        while i < len(tokens):
            n = min(PAGE - self.kv_len[s] % PAGE, len(tokens) - i)
            logits = self.eng.forward(self._batch([(s, tokens[i:i + n])]))
            i += n
        return logits

    def decode(self, seqs: list[int], last_tokens: list[int]) -> torch.Tensor:
        """One step for every sequence; logits [S, vocab]."""
        return self.eng.forward(self._batch([(s, [t]) for s, t in zip(seqs, last_tokens)]))
