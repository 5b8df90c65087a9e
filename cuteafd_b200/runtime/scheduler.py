"""Shared continuous-batching scheduler.

One loop owns every request: admission (queue bound -> KV lease -> prefix lookup / fork -> bind),
chunked prefill time-sliced against decode by ``decode_share``, and decode rounds
(plan drafts -> draft -> settle under the row budget -> verify -> select -> accept -> commit ->
observe -> emit).  A failed device step fails every request of that step with a ``worker`` failure and
quarantines their KV (kernels of the failed step may still be writing it) instead of returning it to the
pool; a failure that happened on the host before anything was launched (no pages left, a malformed batch) and a
per-row sampling error leave the KV intact, so those pages are released.  Readiness is published only after the
backend, the prefix cache, the selector and the draft policy exist.

The engine is behind a ``Backend`` protocol, so the same loop runs on the CUDA engine and on the
CPU oracle backend used by the tests and the fake server.  Counterpart:
rust/crates/cuteafd-daemon/src/shared/qwen/scheduler.rs:103-197 (Backend), :795-1350 (schedule),
:1368-1584 (decode_round), :1459-1473 (failure + quarantine), serve/lanes.rs (lanes).
"""
from __future__ import annotations

import queue
import threading
import time
from dataclasses import dataclass, field
from typing import Any, Protocol

import torch

from . import sampling
from .native import make_reserve
from .speculation import DraftHistory, DrafterSpec, NoDrafter, Plan

FAIL_BAD_REQUEST, FAIL_UNAVAILABLE, FAIL_RETRY, FAIL_WORKER = "bad_request", "unavailable", "retry", "worker"


def _device_failure(e: Exception) -> bool:
    """False for failures raised on the host before a kernel of the step was launched."""
    from ..utils.fault import InjectedFault
    from .paged import OutOfPages
    if isinstance(e, InjectedFault):
        return e.device
    return not isinstance(e, (OutOfPages, ValueError, KeyError, AssertionError))


class Backend(Protocol):
    vocab_size: int
    max_decode_rows: int
    prefill_chunk: int
    total_pages: int

    def open(self, tokens: list[int]) -> tuple[Any, int]: ...                  # (handle, cached prefix length)
    def prefill(self, handle: Any, tokens: list[int], last: bool) -> torch.Tensor | None: ...
    def verify(self, handles: list[Any], rows: list[list[int]]) -> torch.Tensor: ...   # logits [sum(len(rows)), V]
    def commit(self, handle: Any, keep_tokens: int) -> None: ...               # KV length after the round
    def capture(self, handle: Any, kind: str) -> None: ...
    def release(self, handle: Any) -> None: ...
    def quarantine(self, handle: Any) -> None: ...
    def pages_of(self, handle: Any) -> int: ...


@dataclass
class Request:
    prompt: list[int]
    max_tokens: int = 128
    params: sampling.SamplingParams = field(default_factory=sampling.SamplingParams)
    stop_ids: tuple[int, ...] = ()
    speculation: bool = True
    record_rows: bool = False          # probe: keep a hash of every selected logit row
    constraint: Any = None             # TokenConstraint: allowed-token mask applied first in the chain
    stop_texts: tuple = ()             # stop strings longer than one token: matched on the decoded text by the server
    top_logprobs: int = 0              # > 0: keep the chosen token's log-probability and this many alternatives per token
    cold: bool = False                 # probe: do not look the prompt up in the prefix cache
    # probe: teacher-forced scoring.  Run the prompt, record the logits row predicting every prompt token from this index
    # on, end without generating (rust/crates/cuteafd-api/src/openai/probe.rs:50-53).  ``score_want``: per predicted
    # position, token ids whose log-probability to report; ``verify_rows``: width of the decode-shaped scoring steps.
    score_from: int | None = None
    score_want: dict = field(default_factory=dict)
    score_positions: tuple | None = None
    verify_rows: int = 0
    record_state: bool = False         # probe: hash the sequence's persistent state at the prompt and turn frontiers
    media: Any = None                  # list of media spans (prompt position, embedding rows) for ids above the vocabulary
    rid: int = 0
    events: "queue.Queue[tuple]" = field(default_factory=queue.Queue)
    cancelled: threading.Event = field(default_factory=threading.Event)
    arrival: float = 0.0


@dataclass
class Active:
    req: Request
    handle: Any
    cached: int
    prompt_done: int = 0               # prompt tokens whose KV exists (including cached)
    generated: list[int] = field(default_factory=list)
    last_token: int = -1
    kv_len: int = 0
    row_hashes: list[str] = field(default_factory=list)
    spec: dict = field(default_factory=lambda: {"proposed": 0, "accepted": 0, "cycles": 0})
    first_token_at: float = 0.0
    stalled: bool = False
    top_rows: list = field(default_factory=list)   # per selected token: (token, logprob, top ids, top logprobs)
    guard: Any = None                  # RepeatGuard (loop abort), None when the detector is off
    finish_detail: str = ""
    score_rows: list = field(default_factory=list)     # probe ``score_from``: one record per predicted prompt position
    state_hashes: list = field(default_factory=list)   # probe ``record_state``: (frontier, kv length, hash)


@dataclass
class SchedulerStats:
    admitted: int = 0
    packed_steps: int = 0              # prefill steps that carried chunks of more than one prompt
    finished: int = 0
    failed: int = 0
    rejected: int = 0
    prefill_tokens: int = 0
    cached_tokens: int = 0
    decode_rounds: int = 0
    emitted_tokens: int = 0
    verify_rows: int = 0
    verify_row_hist: dict = field(default_factory=dict)
    lane_rounds: dict = field(default_factory=dict)
    stalls: int = 0
    quarantined: int = 0
    loop_aborts: int = 0


class Scheduler:
    def __init__(self, backend: Backend, *, max_active: int = 32, queue_depth: int = 64, queue_wait_s: float = 30.0,
                 decode_share: float = 0.2, drafter=None, draft_control: str = "history", row_budget: int | None = None,
                 eos_ids: tuple[int, ...] = (), decode_lanes: int = 1, loop_abort=None, reserve_chunk_tokens: int = 0,
                 early_end_tokens: int = -1):
        self.be = backend
        from ..utils.fault import NONE
        self.faults = NONE                    # utils.fault.FaultHooks when development fault injection is configured
        # KV pressure: a request that would stall (its top-up is refused) ends with ``length`` once it has produced this
        # many tokens; -1 = off, requests stall and never end early (KV_EARLY_TERMINATION_MIN_OUTPUT_TOKENS)
        self.early_end_tokens = early_end_tokens
        self.loop_abort = loop_abort          # LoopAbortConfig or None (runtime/repeat_guard.py)
        self.trace = None                     # utils.trace.JsonlTrace: one record per decode round when set
        self.watchdog = None                  # utils.diagnostics.StallWatchdog: beaten every step when set
        # Decode lanes: 1 or 2 independent decode batches served in turn on the one engine thread.  A request stays in
        # the lane it was assigned when its prefill finished; each lane keeps its own batch geometry (its own decode
        # graphs).  On a disaggregated deployment lane A's attention overlaps lane B's expert exchange
        # (rust/crates/cuteafd-daemon/src/shared/qwen/scheduler.rs decode lanes; shared-engine.md:181-281).
        self.decode_lanes = max(1, min(2, decode_lanes))
        self._lane_turn = 0
        self.max_active, self.queue_depth, self.queue_wait_s = max_active, queue_depth, queue_wait_s
        self.decode_share = decode_share
        self.waiting: "queue.Queue[Request]" = queue.Queue()
        self.pending: list[Request] = []
        self.prefilling: list[Active] = []
        self.decoding: list[Active] = []
        # page 0 is the reserved zero page; C++ reserve when the library loads.  ``reserve_chunk_tokens``: the decode chunk
        # a request leases beyond its prompt and tops up by (0 = the default of 16 384 tokens)
        self.reserve = (make_reserve(backend.total_pages - 1, reserve_chunk_tokens) if reserve_chunk_tokens > 0
                        else make_reserve(backend.total_pages - 1))
        self.drafter = drafter or NoDrafter()
        self.policy = DraftHistory(self.drafter.spec if hasattr(self.drafter, "spec") else DrafterSpec(0), draft_control)
        self.row_budget = row_budget or backend.max_decode_rows
        self.eos_ids = eos_ids
        self.stats = SchedulerStats()
        self._rid = 0
        self._lock = threading.Lock()
        self._stop = threading.Event()
        self._t_prefill = 0.0
        self._t_decode = 0.0
        self.ready = threading.Event()
        self.ready.set()                      # everything above is built: publish readiness last

    # ---- submission (any thread) ------------------------------------------------------------------
    def submit(self, req: Request) -> Request:
        with self._lock:
            self._rid += 1
            req.rid = self._rid
        req.arrival = time.monotonic()
        # ids at or above the vocabulary are media rows: each must be covered by one of the request's spans
        covered = set()
        for sp in req.media or ():
            covered.update(range(sp.start, sp.start + sp.length))
        V = self.be.vocab_size
        if not req.prompt or any(t < 0 or (t >= V and i not in covered) for i, t in enumerate(req.prompt)) or req.max_tokens < 1:
            req.events.put(("error", FAIL_BAD_REQUEST, "empty prompt, token out of range or max_tokens < 1"))
            self.stats.rejected += 1
            return req
        limit = getattr(self.be, "max_context_tokens", None)
        if limit is not None and len(req.prompt) + req.max_tokens > limit:
            # refused at the door, as a client error: a longer sequence does not fit the per-sequence page table
            req.events.put(("error", FAIL_BAD_REQUEST, f"prompt ({len(req.prompt)} tokens) + max_tokens ({req.max_tokens}) exceeds the "
                                                       f"deployment's context of {limit} tokens"))
            self.stats.rejected += 1
            return req
        if self.waiting.qsize() + len(self.pending) >= self.queue_depth:
            req.events.put(("error", FAIL_RETRY, "admission queue full"))
            self.stats.rejected += 1
            return req
        self.waiting.put(req)
        return req

    # ---- the loop ----------------------------------------------------------------------------------
    def run_forever(self, idle_sleep: float = 0.001) -> None:
        while not self._stop.is_set():
            if not self.step():
                time.sleep(idle_sleep)

    def stop(self) -> None:
        self._stop.set()

    def step(self) -> bool:
        """One scheduling iteration.  Returns False when there was nothing to do."""
        if self.watchdog is not None:
            self.watchdog.beat()
            self.watchdog.busy(len(self.prefilling) + len(self.decoding))
        self._drain_queue()
        self._admit()
        # While both kinds of work exist, decode gets ``decode_share`` of the measured step time and
        # prefill the rest; the shares are tracked with exponentially decayed clocks.
        if self.prefilling and self.decoding:
            total = self._t_prefill + self._t_decode
            do_prefill = total == 0.0 or self._t_decode / total >= self.decode_share
        else:
            do_prefill = bool(self.prefilling)
        t0 = time.monotonic()
        if do_prefill:
            did = self._prefill_packed() if len(self.prefilling) > 1 and hasattr(self.be, "prefill_packed") else self._prefill_one()
            self._t_prefill = 0.9 * self._t_prefill + (time.monotonic() - t0)
            self._t_decode *= 0.9
        elif self.decoding:
            did = self._decode_round()
            self._t_decode = 0.9 * self._t_decode + (time.monotonic() - t0)
            self._t_prefill *= 0.9
        else:
            did = False
        return did

    def _drain_queue(self) -> None:
        while True:
            try:
                self.pending.append(self.waiting.get_nowait())
            except queue.Empty:
                break
        now = time.monotonic()
        keep = []
        for r in self.pending:
            if r.cancelled.is_set():
                # cancelled before it was admitted: it still ends, like a request cancelled in flight, with what it cost
                r.events.put(("done", "cancelled", {"prompt_tokens": len(r.prompt), "completion_tokens": 0, "cached_tokens": 0,
                                                    "speculation": {"proposed": 0, "accepted": 0, "cycles": 0, "request_id": r.rid}}, []))
                continue
            if now - r.arrival > self.queue_wait_s:
                r.events.put(("error", FAIL_RETRY, "queue wait exceeded"))
                self.stats.rejected += 1
            else:
                keep.append(r)
        self.pending = keep

    def _admit(self) -> None:
        while self.pending and len(self.prefilling) + len(self.decoding) < self.max_active:
            req = self.pending[0]
            try:
                handle, cached = self.be.open(req.prompt, cold=True) if (req.cold or req.score_from is not None) else self.be.open(req.prompt)
            except Exception as e:                      # a failed restore is a miss, not an error
                req.events.put(("error", FAIL_UNAVAILABLE, f"open failed: {e}"))
                self.pending.pop(0)
                self.stats.failed += 1
                continue
            lease = self.reserve.lease(req.rid, len(req.prompt), req.max_tokens, shared_pages=cached // 64)
            if lease is None:
                self.be.release(handle)
                if not self.prefilling and not self.decoding:
                    req.events.put(("error", FAIL_RETRY, "request does not fit the KV pool"))
                    self.pending.pop(0)
                    self.stats.rejected += 1
                    continue
                break                                   # wait for running requests to release pages
            self.pending.pop(0)
            if req.media:
                handle.media = req.media
            a = Active(req, handle, cached, prompt_done=cached, kv_len=cached)
            a.guard = self.loop_abort.guard() if self.loop_abort is not None else None
            self.stats.admitted += 1
            self.stats.cached_tokens += cached
            if req.score_from is not None:
                self._score(a)
                continue
            self.prefilling.append(a)

    # ---- probes ------------------------------------------------------------------------------------------
    def _score(self, a: Active) -> None:
        """Teacher-forced scoring of a prompt (a synchronous diagnostic): prefill up to the first scored position, then
        decode-shaped steps of ``verify_rows`` prompt tokens each, recording the row that predicts every prompt token
        from ``score_from`` on.  Nothing is generated and nothing is captured."""
        req, p = a.req, a.req.prompt
        first = max(1, min(int(req.score_from), len(p)))           # token 0 has no predicting row
        width = max(1, min(req.verify_rows or self.be.max_decode_rows, self.be.max_decode_rows))
        keep = None if req.score_positions is None else set(int(x) for x in req.score_positions)

        def record(position: int, row: torch.Tensor) -> None:
            if position >= len(p) or (keep is not None and position not in keep):
                return
            lp = torch.log_softmax(row.float(), dim=-1).cpu()
            rec = {"position": position, "token": int(p[position]), "logprob": float(lp[p[position]]),
                   "hash": sampling.row_hash(row)}
            if req.top_logprobs:
                v, i = lp.topk(min(req.top_logprobs, lp.numel()))
                rec["top_ids"], rec["top_logprobs"] = i.tolist(), v.tolist()
            want = req.score_want.get(position) or req.score_want.get(str(position))
            if want:
                rec["want"] = {int(t): float(lp[int(t)]) for t in want if 0 <= int(t) < lp.numel()}
            a.score_rows.append(rec)

        try:
            logits = None
            while a.prompt_done < first:
                n = min(self.be.prefill_chunk, first - a.prompt_done)
                logits = self.be.prefill(a.handle, p[a.prompt_done:a.prompt_done + n], a.prompt_done + n == first)
                a.prompt_done += n
                self.stats.prefill_tokens += n
            if logits is not None:
                record(first, logits[0] if logits.dim() == 2 else logits)
            pos = a.prompt_done
            while pos < len(p) - 1:                                 # feeding token i gives the row predicting token i + 1
                n = min(width, len(p) - 1 - pos)
                rows = self.be.verify([a.handle], [p[pos:pos + n]])
                self.be.commit(a.handle, pos + n)
                for j in range(n):
                    record(pos + j + 1, rows[j])
                pos += n
                self.stats.verify_rows += n
            a.kv_len = pos
            if req.record_state:
                self._record_state(a, "prompt")
        except Exception as e:
            self._fail([a], f"scoring failed: {e}", device=_device_failure(e))
            return
        self._finish(a, "stop", retain=False)

    def _record_state(self, a: Active, frontier: str) -> None:
        fn = getattr(self.be, "state_hash", None)
        if fn is not None:
            a.state_hashes.append({"frontier": frontier, "kv_len": a.kv_len, "hash": fn(a.handle)})

    # ---- prefill -----------------------------------------------------------------------------------
    PACK_MAX = 8                       # prompts whose chunks may share one prefill step

    def _prefill_packed(self) -> bool:
        """Several short prompts in one forward step: the head request's chunk plus whole chunks of the requests
        behind it while the token budget of a step lasts.  Counterpart: the reference's prefill packing
        (rust/crates/cuteafd-daemon/src/shared/prefill_pipeline.rs)."""
        budget = self.be.prefill_chunk
        group, used = [], 0
        for a in self.prefilling[: self.PACK_MAX]:
            if a.req.cancelled.is_set():
                break
            n = min(budget - used, len(a.req.prompt) - a.prompt_done)
            if n <= 0 or (group and n < len(a.req.prompt) - a.prompt_done and n < 64):
                break                                   # no sliver chunks for the requests behind the head
            group.append((a, n))
            used += n
            if used >= budget:
                break
        if len(group) < 2:
            return self._prefill_one()
        items = [(a.handle, a.req.prompt[a.prompt_done:a.prompt_done + n], a.prompt_done + n == len(a.req.prompt)) for a, n in group]
        try:
            self.faults.hit("BEFORE_PREFILL")
            outs = self.be.prefill_packed(items)
            self.faults.hit("AFTER_SUBMISSION")
        except Exception as e:
            for a, _ in group:
                self.prefilling.remove(a)
            self._fail([a for a, _ in group], f"prefill failed: {e}", device=_device_failure(e))
            return True
        self.stats.packed_steps += 1
        for (a, n), (_, _, last), logits in zip(group, items, outs):
            a.prompt_done += n
            a.kv_len = a.prompt_done
            self.stats.prefill_tokens += n
            if last:
                self.prefilling.remove(a)
                self._safe(lambda a=a: self.be.capture(a.handle, "prompt"))
                if a.req.record_state:
                    self._safe(lambda a=a: self._record_state(a, "prompt"))
                tok = self._select(a, logits[0] if logits.dim() == 2 else logits, len(a.req.prompt))
                a.first_token_at = time.monotonic()
                if tok is None:
                    continue
                if not self._emit(a, [tok]):
                    self.decoding.append(a)
        return True

    def _prefill_one(self) -> bool:
        a = self.prefilling[0]
        if a.req.cancelled.is_set():
            self.prefilling.pop(0)
            if a.prompt_done >= 64:
                self._safe(lambda: self.be.capture(a.handle, "prompt"))     # parked at a chunk boundary
            self._finish(a, None)
            return True
        n = min(self.be.prefill_chunk, len(a.req.prompt) - a.prompt_done)
        chunk = a.req.prompt[a.prompt_done:a.prompt_done + n]
        last = a.prompt_done + n == len(a.req.prompt)
        try:
            self.faults.hit("BEFORE_PREFILL")
            logits = self.be.prefill(a.handle, chunk, last)
            self.faults.hit("AFTER_SUBMISSION")
        except Exception as e:
            self.prefilling.pop(0)
            self._fail([a], f"prefill failed: {e}", device=_device_failure(e))
            return True
        a.prompt_done += n
        a.kv_len = a.prompt_done
        self.stats.prefill_tokens += n
        if last:
            self.prefilling.pop(0)
            self._safe(lambda: self.be.capture(a.handle, "prompt"))
            if a.req.record_state:
                self._safe(lambda: self._record_state(a, "prompt"))
            tok = self._select(a, logits[0] if logits.dim() == 2 else logits, len(a.req.prompt))
            a.first_token_at = time.monotonic()
            if tok is None:
                return True
            if not self._emit(a, [tok]):
                self.decoding.append(a)
        return True

    # ---- decode round -------------------------------------------------------------------------------
    def _decode_round(self) -> bool:
        batch = [a for a in self.decoding if not a.req.cancelled.is_set()]
        for a in self.decoding:
            if a.req.cancelled.is_set():
                self._finish(a, None, retain=False)        # a cancelled decode is not retained
        self.decoding = batch
        if not batch:
            return False
        if self.decode_lanes > 1:
            # serve one lane per round, alternating; a lane with nothing to do yields its turn
            for _ in range(self.decode_lanes):
                lane = self._lane_turn
                self._lane_turn = (self._lane_turn + 1) % self.decode_lanes
                mine = [a for a in batch if a.req.rid % self.decode_lanes == lane]
                if mine:
                    batch = mine
                    self.stats.lane_rounds[lane] = self.stats.lane_rounds.get(lane, 0) + 1
                    break
        # KV top-ups: a request that cannot grow stalls for this round (never truncated)
        runnable = []
        for a in batch:
            need = a.kv_len + 1 + self.policy.spec.block + self.policy.spec.copy
            if self.reserve.needs_top_up(a.req.rid, need) and not self.reserve.top_up(a.req.rid):
                if 0 <= self.early_end_tokens <= len(a.generated):
                    a.finish_detail = "kv_pressure"        # the operator chose a short reply over a stalled one
                    self.decoding.remove(a)
                    self._finish(a, "length")
                    continue
                a.stalled = True
                self.stats.stalls += 1
                continue
            a.stalled = False
            runnable.append(a)
        if not runnable:
            return False
        runnable = runnable[: self.be.max_decode_rows]
        plans: list[Plan] = []
        drafts: list[list[int]] = []
        heads: list[list[float] | None] = []
        for a in runnable:
            room = a.req.max_tokens - len(a.generated) - 1
            use = a.req.speculation and room > 0 and a.req.constraint is None
            plan = self.policy.plan(a.req.rid, room if use else 0)
            toks, scores = (self.drafter.draft(a.req.rid, None, a.last_token, plan.keep) if plan.keep else ([], None))
            plan = self.policy.refine(plan, len(toks), scores)
            toks = toks[:plan.keep]
            extra = self.policy.extend_copy(plan, a.req.prompt + a.generated, toks, a.req.params.greedy) if toks else []
            plans.append(plan)
            drafts.append(toks + extra[: max(0, room - len(toks))])
            heads.append(scores)
        self.policy.settle(plans, self.row_budget)
        drafts = [d[: p.keep + p.copy] for d, p in zip(drafts, plans)]
        # a copied history may contain media rows (ids above the vocabulary): a draft stops before the first one
        V = self.be.vocab_size
        drafts = [d[: next((i for i, t in enumerate(d) if t >= V or t < 0), len(d))] for d in drafts]
        rows = [[a.last_token] + d for a, d in zip(runnable, drafts)]
        # GPU selection when nothing needs the logit rows on the host (grammar masks advance per token on the
        # host; row hashes are taken from the row bytes)
        on_device = hasattr(self.be, "verify_select") and all(
            a.req.constraint is None and not a.req.record_rows and not a.req.top_logprobs for a in runnable)
        picked: list[int] | None = None
        picked_status: list[int] = []
        try:
            self.faults.hit("BEFORE_DECODE")
            if on_device:
                flat_params = [a.req.params for a, r in zip(runnable, rows) for _ in r]
                flat_pos = [len(a.req.prompt) + len(a.generated) + j for a, r in zip(runnable, rows) for j in range(len(r))]
                picked, picked_status = self.be.verify_select([a.handle for a in runnable], rows, flat_params, flat_pos)
                logits = None
            else:
                logits = self.be.verify([a.handle for a in runnable], rows)
            self.faults.hit("AFTER_SUBMISSION")
        except Exception as e:
            self.decoding = [a for a in self.decoding if a not in runnable]
            self._fail(runnable, f"decode step failed: {e}", device=_device_failure(e))
            return True
        self.stats.decode_rounds += 1
        n_rows = sum(len(r) for r in rows)
        self.stats.verify_rows += n_rows
        self.stats.verify_row_hist[n_rows] = self.stats.verify_row_hist.get(n_rows, 0) + 1
        off = 0
        done: list[Active] = []
        t_round = time.monotonic()
        acc_round: list[int] = []
        for a, plan, d, r, hs in zip(runnable, plans, drafts, rows, heads):
            sel = []
            bad = False
            for j in range(len(r)):
                # row j is drawn at absolute position (tokens so far) + j: layout cannot change a draw
                if picked is not None:
                    t = picked[off + j] if picked_status[off + j] == 0 else None
                else:
                    t = self._select(a, logits[off + j], len(a.req.prompt) + len(a.generated) + j, emit_error=False)
                if t is None:
                    bad = True
                    break
                sel.append(t)
                if j < len(d) and d[j] != t:
                    break                                  # later rows are conditioned on a rejected draft
            off += len(r)
            if bad:
                self._fail([a], "non-finite logits")
                done.append(a)
                continue
            n_acc, bonus = sampling.accept_prefix(sel, d)
            new = d[:n_acc] + [bonus]
            mtp = getattr(self.be, "last_mtp", None)
            if picked is not None and mtp is not None and hasattr(self.drafter, "offer"):
                # the MTP depth ran on this step's rows: the row that supplied the bonus token drafts the token after it
                row = off - len(r) + n_acc
                if row < len(mtp):
                    self.drafter.offer(a.req.rid, [mtp[row]])
            a.kv_len += 1 + n_acc                           # last_token + accepted drafts now have KV
            self.be.commit(a.handle, a.kv_len)
            a.spec["proposed"] += len(d)                    # before the emission: a reply that ends in this round reports it too
            a.spec["accepted"] += n_acc
            a.spec["cycles"] += 1
            stopped = self._emit(a, new)
            self.policy.observe(plan, n_acc, censored=stopped and n_acc < len(d), head_scores=hs)
            if not stopped:                               # a finished request's drafter state is already gone
                self.drafter.accept(a.req.rid, new)
            acc_round.append(n_acc)
            if stopped:
                done.append(a)
        if self.trace is not None:
            self.trace.record(round=self.stats.decode_rounds, requests=[a.req.rid for a in runnable], rows=n_rows,
                              proposed=[len(d) for d in drafts], kept=[p.keep for p in plans], copied=[p.copy for p in plans],
                              accepted=acc_round, on_device=picked is not None, finished=len(done),
                              select_ms=round((time.monotonic() - t_round) * 1e3, 3))
        self.decoding = [a for a in self.decoding if a not in done]
        return True

    # ---- helpers -------------------------------------------------------------------------------------
    def _select(self, a: Active, row: torch.Tensor, position: int, emit_error: bool = True) -> int | None:
        try:
            c = a.req.constraint
            tok = sampling.select_token(row, a.req.params, position, c.mask() if c is not None else None)
            if c is not None:
                c.advance(tok)
        except sampling.SamplingError as e:
            if emit_error:
                self._fail([a], str(e))
            return None
        if a.req.record_rows:
            a.row_hashes.append(sampling.row_hash(row))
        if a.req.top_logprobs:
            lp = torch.log_softmax(row.float(), dim=-1)
            v, i = lp.topk(min(a.req.top_logprobs, lp.numel()))
            a.top_rows.append((int(tok), float(lp[tok]), i.tolist(), v.tolist()))
        return tok

    def _emit(self, a: Active, toks: list[int]) -> bool:
        """Append tokens, stream them, return True when the request is finished."""
        finish = None
        out = []
        for t in toks:
            a.generated.append(t)
            out.append(t)
            if t in a.req.stop_ids or t in self.eos_ids:
                finish = "stop"
                break
            if a.req.constraint is not None and a.req.constraint.finished():
                finish = "stop"
                break
            if len(a.generated) >= a.req.max_tokens:
                finish = "length"
                break
            if a.guard is not None and a.guard.push(t):
                finish, a.finish_detail = "length", "repetition"      # an exact loop ends like max_tokens
                self.stats.loop_aborts += 1
                break
        if len(a.generated) == len(out) and hasattr(self.drafter, "begin") and a.req.speculation:
            # the reply's first token: a drafter that keeps per-request state (history, a draft model's KV) starts here
            self._safe(lambda: self.drafter.begin(a.req.rid, a.req.prompt, a.generated[0]))
        a.last_token = a.generated[-1]
        self.stats.emitted_tokens += len(out)
        a.req.events.put(("tokens", out))
        if finish:
            self._finish(a, finish)
            return True
        return False

    def _finish(self, a: Active, reason: str | None, retain: bool = True) -> None:
        if reason is not None and retain:
            self._safe(lambda: self.be.capture(a.handle, "turn"))
            if a.req.record_state:
                self._safe(lambda: self._record_state(a, "turn"))
        self._safe(lambda: self.be.release(a.handle))
        self.reserve.release(a.req.rid)
        self.policy.forget(a.req.rid)
        if hasattr(self.drafter, "forget"):
            self._safe(lambda: self.drafter.forget(a.req.rid))
        if reason is not None:
            usage = {"prompt_tokens": len(a.req.prompt), "completion_tokens": len(a.generated), "cached_tokens": a.cached,
                     "speculation": dict(a.spec, request_id=a.req.rid)}
            if a.finish_detail:
                usage["finish_detail"] = a.finish_detail
            if a.req.score_from is not None:
                usage["score_rows"] = a.score_rows
            if a.state_hashes:
                usage["state_hashes"] = a.state_hashes
            if a.req.top_logprobs:
                # rows were kept per selection; a reply cut by a stop or a limit keeps the rows of the emitted tokens
                usage["top_rows"] = a.top_rows[: len(a.generated)]
            a.req.events.put(("done", reason, usage, list(a.row_hashes)))
            self.stats.finished += 1
        else:
            # a cancelled request still says what it cost (a stop string ends a reply by cancelling it)
            a.req.events.put(("done", "cancelled", {"prompt_tokens": len(a.req.prompt), "completion_tokens": len(a.generated),
                                                    "cached_tokens": a.cached, "speculation": dict(a.spec, request_id=a.req.rid)}, []))

    def _fail(self, actives: list[Active], msg: str, device: bool = False) -> None:
        """``device``: the step may have reached the GPU, so the requests' pages are quarantined (kept allocated, never
        handed out again) rather than released (rust/crates/cuteafd-daemon/src/shared/qwen/scheduler.rs:1459-1473)."""
        for a in actives:
            if device:
                self._safe(lambda a=a: self.be.quarantine(a.handle))
                self.stats.quarantined += 1
            else:
                try:
                    self.be.release(a.handle)
                except Exception:
                    self._safe(lambda a=a: self.be.quarantine(a.handle))
                    self.stats.quarantined += 1
            self.reserve.release(a.req.rid)
            self.policy.forget(a.req.rid)
            if hasattr(self.drafter, "forget"):
                self._safe(lambda a=a: self.drafter.forget(a.req.rid))
            a.req.events.put(("error", FAIL_WORKER, msg))
            self.stats.failed += 1

    @staticmethod
    def _safe(fn) -> None:
        try:
            fn()
        except Exception:
            pass

    def lanes(self) -> list[dict]:
        """One row per request in flight (console view; read from another thread, so lists are copied first)."""
        now = time.monotonic()
        out = []
        for phase, group in (("prefill", list(self.prefilling)), ("decode", list(self.decoding))):
            for a in group:
                prop = a.spec["proposed"]
                out.append({"rid": a.req.rid, "phase": "stalled" if a.stalled else phase,
                            "lane": a.req.rid % self.decode_lanes, "prompt_tokens": len(a.req.prompt),
                            "prompt_done": a.prompt_done, "cached_tokens": a.cached, "generated": len(a.generated),
                            "max_tokens": a.req.max_tokens, "kv_len": a.kv_len, "cycles": a.spec["cycles"],
                            "acceptance": round(a.spec["accepted"] / prop, 3) if prop else None,
                            "tokens_per_cycle": round(len(a.generated) / a.spec["cycles"], 2) if a.spec["cycles"] else None,
                            "age_s": round(now - a.req.arrival, 2),
                            "ttft_s": round(a.first_token_at - a.req.arrival, 3) if a.first_token_at else None})
        return out

    def snapshot(self) -> dict:
        s = self.stats
        return {"active": len(self.decoding), "prefilling": len(self.prefilling), "queued": len(self.pending) + self.waiting.qsize(),
                "admitted": s.admitted, "finished": s.finished, "failed": s.failed, "rejected": s.rejected,
                "prefill_tokens": s.prefill_tokens, "cached_tokens": s.cached_tokens, "decode_rounds": s.decode_rounds,
                "emitted_tokens": s.emitted_tokens, "verify_rows": s.verify_rows, "stalls": s.stalls,
                "quarantined": s.quarantined, "loop_aborts": s.loop_aborts, "packed_steps": s.packed_steps,
                "verify_row_hist": dict(s.verify_row_hist), "lane_rounds": dict(s.lane_rounds),
                "time_share": {"prefill": round(self._t_prefill, 4), "decode": round(self._t_decode, 4)},
                "draft_policy": dict(self.policy.lifetime),
                "kv": {"total_pages": self.reserve.total, "leased_pages": self.reserve.leased}}


def collect(req: Request, timeout: float = 60.0) -> dict:
    """Block until a request finishes; returns {"tokens", "finish", "usage", "error", "row_hashes"}."""
    toks: list[int] = []
    t0 = time.monotonic()
    while True:
        try:
            ev = req.events.get(timeout=max(0.01, timeout - (time.monotonic() - t0)))
        except queue.Empty:
            return {"tokens": toks, "finish": None, "usage": {}, "error": ("timeout", "no event"), "row_hashes": []}
        if ev[0] == "tokens":
            toks.extend(ev[1])
        elif ev[0] == "done":
            return {"tokens": toks, "finish": ev[1], "usage": ev[2], "error": None, "row_hashes": ev[3]}
        elif ev[0] == "error":
            return {"tokens": toks, "finish": None, "usage": {}, "error": (ev[1], ev[2]), "row_hashes": []}
