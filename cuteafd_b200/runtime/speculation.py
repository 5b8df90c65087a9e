"""History-adaptive speculative decoding: how many drafted positions each request verifies, the
history "copy" track, and the drafter interface (MTP head, remote, none).

Policy (per request i, drafted position k):
    p_ik = (s_ik + m * g_k) / (t_ik + m)
where s/t are accepted/reached counts over the request's last 8 verify rounds, g_k the server-wide
acceptance at k over the last 256 rounds that reached k, and m a prior strength of 8 that fades to
zero after the request has completed 3 rounds.  Positions are kept while p_ik > 0.3, each judged
alone; one position past the stop is always explored (up to the drafter's block) so estimates
cannot lock low.  A drafter with a confidence head may skip the explore position when its
calibrated probability is below 0.3.  When the round exceeds the verify-row budget, positions are
granted across requests highest-probability first, each request keeping a prefix of its plan.

Copy track: when the last 4-8 emitted tokens occurred earlier in the request's history, the
tokens that followed that earlier occurrence are proposed as extra draft positions (greedy
requests only, at most 32, needs 3 agreeing drafts and 7 anchored tokens); its cold rate 0.25 is
below the keep cut so a cold copy verifies only its explored first row.

Counterpart: rust/crates/cuteafd-core/src/draft_history.rs:1-120 (policy, constants),
rust/crates/cuteafd-daemon/src/shared/draft/copy.rs:8-46 (copy window),
rust/crates/cuteafd-daemon/src/shared/speculation.rs (drafter kinds).
"""
from __future__ import annotations

import math
from collections import deque
from dataclasses import dataclass, field
from typing import Protocol

REQUEST_WINDOW = 8
SERVER_WINDOW = 256
PRIOR_STRENGTH = 8.0
FADE_ROUNDS = 3
KEEP_CUT = 0.3
SKIP_CUT = 0.3
NEURAL_COLD_RATE = 1.0
COPY_COLD_RATE = 0.25
COPY_MIN_SUFFIX, COPY_MAX_SUFFIX, COPY_MAX_EXTRA = 4, 8, 32
COPY_MIN_AGREE, COPY_MIN_ANCHORED = 3, 7


@dataclass(frozen=True)
class DrafterSpec:
    block: int            # most positions one draft pass proposes
    head: bool = False    # trained confidence head
    copy: int = 0         # most copy positions past the neural draft


class _Track:
    """Windows for one kind of position (neural or copy)."""

    def __init__(self, cold: float):
        self.cold = cold
        self.server: dict[int, deque] = {}                      # k -> last outcomes (1/0) that reached k

    def server_rate(self, k: int) -> float:
        w = self.server.get(k)
        return self.cold if not w else sum(w) / len(w)

    def observe(self, k: int, accepted: bool) -> None:
        self.server.setdefault(k, deque(maxlen=SERVER_WINDOW)).append(1 if accepted else 0)


@dataclass
class _RequestState:
    rounds: int = 0
    neural: deque = field(default_factory=lambda: deque(maxlen=REQUEST_WINDOW))   # per round: (reached, accepted) counts by position
    copy: deque = field(default_factory=lambda: deque(maxlen=REQUEST_WINDOW))


@dataclass
class PlattFit:
    """Online logistic calibration of a head score: p = sigmoid(a * score + b)."""
    a: float = 1.0
    b: float = 0.0
    lr: float = 0.05
    n: int = 0

    def prob(self, score: float) -> float:
        z = max(-30.0, min(30.0, self.a * score + self.b))
        return 1.0 / (1.0 + math.exp(-z))

    def update(self, score: float, accepted: bool) -> None:
        err = self.prob(score) - (1.0 if accepted else 0.0)
        self.a -= self.lr * err * score
        self.b -= self.lr * err
        self.n += 1


@dataclass
class Plan:
    rid: int
    keep: int                 # neural positions to verify (including the explored one)
    explore: int | None       # index of the explored position, None when the block is exhausted
    probs: list[float]
    copy: int = 0             # copy positions appended after the neural ones
    skipped_explore: bool = False


class DraftHistory:
    def __init__(self, spec: DrafterSpec, control: str = "history", fixed: int = 0):
        self.spec, self.control, self.fixed = spec, control, fixed
        self.neural, self.copy = _Track(NEURAL_COLD_RATE), _Track(COPY_COLD_RATE)
        self.req: dict[int, _RequestState] = {}
        self.heads: dict[int, PlattFit] = {}
        self.lifetime = {"rounds": 0, "proposed": 0, "accepted": 0, "explore_skips": 0, "budget_cuts": 0}

    def _p(self, st: _RequestState, window: deque, track: _Track, k: int) -> float:
        s = sum(r[1].get(k, 0) for r in window)
        t = sum(r[0].get(k, 0) for r in window)
        m = PRIOR_STRENGTH * max(0.0, 1.0 - st.rounds / FADE_ROUNDS)
        if t + m == 0:
            return float("nan")                                 # unknown: becomes the explored stop
        return (s + m * track.server_rate(k)) / (t + m)

    # ---- 1. before the draft pass ---------------------------------------------------------------
    def plan(self, rid: int, room: int) -> Plan:
        """How many neural positions to draft/verify for ``rid`` (``room`` caps by max_tokens, KV ...)."""
        st = self.req.setdefault(rid, _RequestState())
        block = max(0, min(self.spec.block, room))
        if self.control == "off" or block == 0:
            return Plan(rid, 0, None, [])
        if self.control == "fixed":
            n = min(self.fixed, block)
            return Plan(rid, n, None, [1.0] * n)
        probs, keep = [], 0
        for k in range(block):
            p = self._p(st, st.neural, self.neural, k)
            probs.append(p)
            if not (p > KEEP_CUT):                              # also stops on NaN (unknown)
                break
            keep += 1
        explore = keep if keep < block else None
        return Plan(rid, keep + (1 if explore is not None else 0), explore, probs)

    # ---- 2. after the draft pass: head scores -----------------------------------------------------
    def refine(self, plan: Plan, proposed: int, head_scores: list[float] | None = None) -> Plan:
        plan.keep = min(plan.keep, proposed)
        if plan.explore is not None and plan.explore >= plan.keep:
            plan.explore = None
        if self.spec.head and head_scores and plan.explore is not None and plan.explore < len(head_scores):
            fit = self.heads.setdefault(plan.explore, PlattFit())
            if fit.n >= 16 and fit.prob(head_scores[plan.explore]) < SKIP_CUT:
                plan.keep = plan.explore
                plan.skipped_explore = True
                self.lifetime["explore_skips"] += 1
        return plan

    # ---- 3. history copy ----------------------------------------------------------------------------
    def extend_copy(self, plan: Plan, history: list[int], draft: list[int], greedy: bool) -> list[int]:
        """Tokens to append after the neural draft (possibly empty)."""
        if not greedy or not self.spec.copy:
            return []
        cont = copy_continuation(history, draft[:plan.keep])
        if not cont:
            return []
        st = self.req.setdefault(plan.rid, _RequestState())
        n = 0
        for k in range(min(len(cont), self.spec.copy, COPY_MAX_EXTRA)):
            p = self._p(st, st.copy, self.copy, k)
            if not (p > KEEP_CUT):
                break
            n += 1
        n = min(len(cont), n + 1)                                # one explored copy position
        plan.copy = n
        return cont[:n]

    # ---- 4. verify-row budget -----------------------------------------------------------------------
    def settle(self, plans: list[Plan], row_budget: int) -> list[Plan]:
        """Each request always gets its one target row; drafted rows are granted by probability."""
        rows = sum(1 + p.keep + p.copy for p in plans)
        if rows <= row_budget:
            return plans
        self.lifetime["budget_cuts"] += 1
        cand = []
        for p in plans:
            for k in range(p.keep + p.copy):
                pr = p.probs[k] if k < len(p.probs) and p.probs[k] == p.probs[k] else 0.0
                cand.append((pr, -k, p.rid))
        grants = {p.rid: 0 for p in plans}
        budget = max(0, row_budget - len(plans))
        # a request keeps a prefix: position k is granted only after k-1
        for pr, negk, rid in sorted(cand, reverse=True):
            if budget == 0:
                break
            if grants[rid] == -negk:
                grants[rid] += 1
                budget -= 1
        for p in plans:
            g = grants[p.rid]
            p.copy = max(0, min(p.copy, g - p.keep))
            p.keep = min(p.keep, g)
        return plans

    # ---- 5. outcome -----------------------------------------------------------------------------------
    def observe(self, plan: Plan, accepted: int, censored: bool = False, head_scores: list[float] | None = None) -> None:
        """``accepted`` drafts were accepted out of plan.keep + plan.copy verified; ``censored`` when
        the round stopped for another reason (stop token, limit) right after the accepted prefix."""
        st = self.req.setdefault(plan.rid, _RequestState())
        n_neural = min(accepted, plan.keep)
        reached_n, acc_n = {}, {}
        for k in range(plan.keep):
            if k > n_neural or (k == n_neural and censored):
                break
            reached_n[k] = 1
            ok = k < n_neural
            acc_n[k] = 1 if ok else 0
            self.neural.observe(k, ok)
            if head_scores and k < len(head_scores) and self.spec.head:
                self.heads.setdefault(k, PlattFit()).update(head_scores[k], ok)
        if plan.skipped_explore and n_neural == plan.keep and not censored:
            k = plan.keep                                         # a skipped explore is booked as a miss
            reached_n[k], acc_n[k] = 1, 0
            self.neural.observe(k, False)
        st.neural.append((reached_n, acc_n))
        if plan.copy and n_neural == plan.keep:
            n_copy = accepted - plan.keep
            reached_c, acc_c = {}, {}
            for k in range(plan.copy):
                if k > n_copy or (k == n_copy and censored):
                    break
                reached_c[k] = 1
                acc_c[k] = 1 if k < n_copy else 0
                self.copy.observe(k, k < n_copy)
            st.copy.append((reached_c, acc_c))
        st.rounds += 1
        self.lifetime["rounds"] += 1
        self.lifetime["proposed"] += plan.keep + plan.copy
        self.lifetime["accepted"] += accepted

    def forget(self, rid: int) -> None:
        self.req.pop(rid, None)


def copy_continuation(history: list[int], draft: list[int]) -> list[int]:
    """Continuation of the latest earlier occurrence of the last 4..8 tokens of history+draft.

    Needs at least COPY_MIN_AGREE agreeing draft tokens and COPY_MIN_ANCHORED anchored tokens
    (suffix + agreement) before anything is proposed."""
    if len(draft) < COPY_MIN_AGREE:
        return []
    seq = history + draft
    for n in range(COPY_MAX_SUFFIX, COPY_MIN_SUFFIX - 1, -1):
        if len(history) < n + 1:
            continue
        suffix = history[-n:]
        for start in range(len(history) - n - 1, -1, -1):
            if history[start:start + n] == suffix:
                follow = history[start + n:]
                agree = 0
                for a, b in zip(follow, draft):
                    if a != b:
                        break
                    agree += 1
                if agree >= COPY_MIN_AGREE and agree == len(draft) and n + agree >= COPY_MIN_ANCHORED:
                    return follow[agree:agree + COPY_MAX_EXTRA]
                break
    return []


class Drafter(Protocol):
    spec: DrafterSpec

    def draft(self, rid: int, last_hidden, last_token: int, n: int) -> tuple[list[int], list[float] | None]: ...
    def accept(self, rid: int, accepted_tokens: list[int]) -> None: ...


class NoDrafter:
    spec = DrafterSpec(block=0)

    def draft(self, rid, last_hidden, last_token, n):
        return [], None

    def accept(self, rid, accepted_tokens):
        return None


class NgramDrafter:
    """Model-free drafter: proposes the continuation of the last occurrence of the current suffix
    (useful on CPU tests and as the "history" baseline for repetitive text)."""

    def __init__(self, block: int = 4, n: int = 3):
        self.spec = DrafterSpec(block=block, head=False, copy=COPY_MAX_EXTRA)
        self.n = n
        self.hist: dict[int, list[int]] = {}

    def draft(self, rid, last_hidden, last_token, n):
        h = self.hist.get(rid, [])
        if len(h) < self.n + 1:
            return [], None
        suf = h[-self.n:]
        for s in range(len(h) - self.n - 1, -1, -1):
            if h[s:s + self.n] == suf:
                return h[s + self.n:s + self.n + n], None
        return [], None

    def begin(self, rid, prompt, first_token):
        """The request's history starts with its prompt (suffixes of the reply are looked up in it too)."""
        self.hist[rid] = list(prompt) + [first_token]

    def accept(self, rid, accepted_tokens):
        self.hist.setdefault(rid, []).extend(accepted_tokens)

    def forget(self, rid):
        self.hist.pop(rid, None)


class ModelDrafter:
    """A small draft model proposes the block: ``draft`` runs it greedily for up to ``n`` tokens from the request's
    last token, ``accept`` rewinds its KV to the tokens the target kept and feeds what the target chose instead.
    Verification decides, so the reply is the target's whatever the draft model says; a draft model that agrees with
    the target k tokens ahead turns k + 1 target steps into one.

    ``step(tokens, kv) -> logits [len(tokens), vocab]`` and ``new_kv()`` are the draft model (here the oracle decoder
    over a small checkpoint; an engine with the same two calls plugs in the same way).  ``scores`` are the draft
    model's probabilities of its own picks, which the history policy can use as head confidence.

    Counterpart: the reference's dSpark block drafter (a small Qwen3 backbone beside the target,
    rust/crates/cuteafd-daemon/src/shared/speculation/)."""

    def __init__(self, step, new_kv, block: int = 4, vocab_size: int | None = None):
        self.spec = DrafterSpec(block=block, head=True, copy=COPY_MAX_EXTRA)
        self.step, self.new_kv, self.vocab = step, new_kv, vocab_size
        self.state: dict[int, dict] = {}
        self.drafted = 0

    @staticmethod
    def from_oracle(cfg, params, block: int = 4, parallel: bool = False) -> "ModelDrafter":
        import torch

        from ..ref.model import KvState, RefDecoder
        dec = RefDecoder(cfg, params)

        def step(tokens, kv, all_rows: bool = False):
            with torch.no_grad():
                return dec.forward(torch.tensor(tokens, dtype=torch.long), kv)
        return (BlockModelDrafter if parallel else ModelDrafter)(step, lambda: KvState(cfg), block, cfg.vocab_size)

    @staticmethod
    def from_engine(engine, num_pages: int, max_pages_per_seq: int, block: int = 4, parallel: bool = False) -> "ModelDrafter":
        """The draft model is a CUDA engine (a small checkpoint of the same vocabulary on the same GPU) with its own
        paged KV.  ``parallel``: the block drafter (one pass per block, see ``BlockModelDrafter``)."""
        m = EngineDraftModel(engine, num_pages, max_pages_per_seq)
        cls = BlockModelDrafter if parallel else ModelDrafter
        d = cls(m.step, m.new_kv, block, engine.cfg.vocab_size)
        d.model = m
        return d

    def begin(self, rid, prompt, first_token):
        kv = self.new_kv()
        toks = [t if self.vocab is None or t < self.vocab else 0 for t in prompt]      # media rows: the draft model sees a filler
        self.step(toks, kv)
        self.state[rid] = {"kv": kv, "base": len(toks), "pending": first_token, "fed": []}

    def draft(self, rid, last_hidden, last_token, n):
        st = self.state.get(rid)
        if st is None or n <= 0:
            return [], None
        import torch
        if st["fed"]:                                   # a draft nobody settled (the plan dropped it): rewind first
            st["kv"].truncate(st["base"])
            st["fed"] = []
        cur, toks, scores = st["pending"], [], []
        for _ in range(n):
            lp = torch.log_softmax(self.step([cur], st["kv"])[-1].float(), dim=-1)
            st["fed"].append(cur)
            cur = int(lp.argmax())
            toks.append(cur)
            scores.append(float(lp[cur].exp()))
        self.drafted += len(toks)
        return toks, scores

    def accept(self, rid, accepted_tokens):
        st = self.state.get(rid)
        if st is None or not accepted_tokens:
            return
        want = [st["pending"]] + list(accepted_tokens[:-1])
        fed = st["fed"]
        common = 0
        while common < min(len(fed), len(want)) and fed[common] == want[common]:
            common += 1
        st["kv"].truncate(st["base"] + common)
        if want[common:]:
            self.step([t if self.vocab is None or t < self.vocab else 0 for t in want[common:]], st["kv"])
        st["base"] += len(want)
        st["pending"], st["fed"] = accepted_tokens[-1], []

    def forget(self, rid):
        self.state.pop(rid, None)


class BlockModelDrafter(ModelDrafter):
    """Block drafter: the whole block comes out of ONE pass of the draft model.  The pass runs over the request's last
    token followed by mask tokens; row j's argmax is the draft of position j + 1, so positions past the first are
    predicted from mask inputs and whatever the draft model's attention makes of the context (the way the reference's
    dSpark / DFlash2 block drafters denoise a masked block in a single forward,
    rust/crates/cuteafd-daemon/src/shared/speculation/block_dspark.rs:1-60, dflash.rs:1-27).  The mask rows' K/V is
    dropped after the pass; only the real token's stays.  One draft-model launch chain per round instead of ``block``."""

    def __init__(self, step, new_kv, block: int = 4, vocab_size: int | None = None, mask_token: int | None = None):
        super().__init__(step, new_kv, block, vocab_size)
        self.mask_token = mask_token if mask_token is not None else (vocab_size - 1 if vocab_size else 0)
        self.passes = 0

    def draft(self, rid, last_hidden, last_token, n):
        st = self.state.get(rid)
        if st is None or n <= 0:
            return [], None
        import torch
        if st["fed"]:
            st["kv"].truncate(st["base"])
            st["fed"] = []
        rows = [st["pending"]] + [self.mask_token] * (n - 1)
        lp = torch.log_softmax(self.step(rows, st["kv"], all_rows=True).float(), dim=-1)
        self.passes += 1
        st["kv"].truncate(st["base"] + 1)               # the mask rows' K/V means nothing: keep the real token's
        st["fed"] = [st["pending"]]
        toks = lp.argmax(dim=-1).tolist()
        self.drafted += len(toks)
        return toks, [float(lp[j, t].exp()) for j, t in enumerate(toks)]


class EngineDraftModel:
    """``step`` / ``new_kv`` of ``ModelDrafter`` on a CUDA engine: one sequence of the engine's paged cache per request,
    tokens appended as prompt-style chunks (causal inside the chunk, the cache before it), logits of the last row or
    of every row back on the host."""

    def __init__(self, engine, num_pages: int, max_pages_per_seq: int, chunk: int = 256):
        from .generate import StepBuffers
        from .native import make_pool
        from .paged import SequenceTable
        self.eng, self.max_pages = engine, max_pages_per_seq
        self.pool = make_pool(num_pages)
        self.table = SequenceTable(self.pool)
        self.chunk = min(chunk, engine.max_tokens)
        self.buf = StepBuffers(self.chunk, 1, max_pages_per_seq, engine.device)
        self.steps = 0

    class _Seq:
        def __init__(self, owner):
            self.owner, self.seq = owner, owner.table.new()

        def truncate(self, length: int) -> None:
            self.owner.table.truncate(self.seq, length)

        def __del__(self):
            try:
                self.owner.table.free(self.seq)
            except Exception:                            # noqa: BLE001 - interpreter shutdown
                pass

    def new_kv(self):
        return EngineDraftModel._Seq(self)

    def step(self, tokens, kv, all_rows: bool = False):
        import torch

        from ..models.gqa_moe import Batch
        seq, b, out = kv.seq, self.buf, None
        rows_cap = self.eng.logits.shape[0]
        for c0 in range(0, len(tokens), self.chunk):
            part = tokens[c0:c0 + self.chunk]
            start, n = seq.kv_len, len(part)
            self.table.reserve(seq, start + n, copy_page=lambda s, d: self.eng.kv.copy_page(s, d))
            b.tokens[0][:n] = torch.tensor(part, dtype=torch.int32)
            b.positions[0][:n] = torch.arange(start, start + n, dtype=torch.int32)
            b.slots[0][:n] = torch.tensor(self.table.slots(seq, start, n), dtype=torch.int32)
            pt = b.page_table[0].view(1, self.max_pages)
            pt.zero_()
            pt[0, :len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
            b.seq_lens[0][0] = start + n
            b.q_start[0][0], b.q_start[0][1] = 0, n
            b.last_rows[0][0] = n - 1
            b.upload()
            every = all_rows and n <= rows_cap
            batch = Batch(b.tokens[1][:n], b.positions[1][:n], b.slots[1][:n], b.page_table[1].view(1, self.max_pages),
                          b.seq_lens[1][:1], b.q_start[1][:2], n, True, None if every else b.last_rows[1][:1], fresh=start == 0)
            out = self.eng.forward(batch)
            seq.tokens.extend(part)
            seq.kv_len = start + n
            self.steps += 1
        return out.float().cpu()


class MtpDrafter:
    """Native multi-token-prediction drafter (depth 1).  The engine runs its MTP depth right after every verify step
    on the rows just scored, pairing each row's final hidden state with the token selected for it, so the draft for
    the next step is ready when the step returns; the backend hands it over with ``offer``.  A draft is consumed by
    the next ``draft`` call; verification decides, so a stale or missing draft costs speed, never correctness.
    (The reference's "recurrent" block drafter, rust/crates/cuteafd-daemon/src/shared/speculation/recurrent.rs:18-40.)"""

    def __init__(self, block: int = 1):
        self.spec = DrafterSpec(block=block, head=False, copy=COPY_MAX_EXTRA)
        self.pending: dict[int, list[int]] = {}
        self.offered = 0

    def offer(self, rid: int, tokens: list[int]) -> None:
        self.pending[rid] = list(tokens)
        self.offered += len(tokens)

    def draft(self, rid, last_hidden, last_token, n):
        toks = self.pending.pop(rid, [])
        return toks[:n], None

    def accept(self, rid, accepted_tokens):
        pass

    def forget(self, rid: int) -> None:
        self.pending.pop(rid, None)
