"""Synchronous generation driver: chunked prefill and batched decode over the paged KV cache,
with the decode step captured in a CUDA graph per batch size.

This is the user-facing "run this batch" layer under the scheduler: step inputs are staged in
pinned host memory and copied to fixed device buffers each step; the selected tokens come back
with one device-to-host read.  The reference's equivalent is its decode graph cache keyed by
exact geometry (rust/crates/cuteafd-daemon/src/shared/decode_graph.rs; bank keys in
rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2208-2210) with an eager fallback.
"""
from __future__ import annotations

import torch

from ..models.gqa_moe import Batch
from .paged import PAGE, PagePool, Sequence, SequenceTable


class StepBuffers:
    """Pinned host staging + device buffers for one step shape (max T tokens, S sequences).

    Callers fill the ``[0]`` (host) views and call ``upload``.  The copy to the device is asynchronous, and the GPU may
    be a whole prompt chunk behind the host, so the bytes it reads must not be the ones the caller fills next:
    ``upload`` snapshots the staging into one of two pinned in-flight buffers (a host memcpy of a few KB) and copies
    from there; an in-flight buffer is reused only after the copy that read it has completed."""

    def __init__(self, max_tokens: int, max_seqs: int, max_pages: int, device: torch.device):
        self.max_tokens, self.max_seqs, self.max_pages = max_tokens, max_seqs, max_pages
        n = 3 * max_tokens + max_seqs * max_pages + max_seqs + (max_seqs + 1) + max_seqs
        self.host = torch.zeros(n, dtype=torch.int32).pin_memory() if device.type == "cuda" else torch.zeros(n, dtype=torch.int32)
        self.dev = torch.zeros(n, dtype=torch.int32, device=device)
        self._inflight = [torch.zeros(n, dtype=torch.int32).pin_memory() for _ in range(2)] if device.type == "cuda" else []
        self._sent = [torch.cuda.Event() for _ in self._inflight]
        self._recorded = [False] * len(self._inflight)
        self._turn = 0
        o = 0

        def take(k: int):
            nonlocal o
            v = (self.host[o:o + k], self.dev[o:o + k])
            o += k
            return v

        self.tokens, self.positions, self.slots = take(max_tokens), take(max_tokens), take(max_tokens)
        self.page_table = take(max_seqs * max_pages)
        self.seq_lens, self.q_start, self.last_rows = take(max_seqs), take(max_seqs + 1), take(max_seqs)
        self.bytes = n * 4

    def upload(self) -> int:
        if not self._inflight:
            self.dev.copy_(self.host)
            return self.bytes
        k = self._turn
        self._turn = (k + 1) % len(self._inflight)
        if self._recorded[k]:
            self._sent[k].synchronize()               # the copy that last read this buffer (two uploads ago) is done
        self._inflight[k].copy_(self.host)
        self.dev.copy_(self._inflight[k], non_blocking=True)
        self._sent[k].record()
        self._recorded[k] = True
        return self.bytes


class Generator:
    def __init__(self, engine, pool: PagePool, max_pages_per_seq: int, max_seqs: int, prefill_chunk: int = 8192,
                 use_graphs: bool = True, max_graphs: int = 16):
        self.engine, self.pool = engine, pool
        self.max_graphs = max_graphs          # decode graphs kept (exact batch size is the key); least recently used goes first
        self.table = SequenceTable(pool)
        self.device = engine.device
        self.max_pages, self.max_seqs, self.chunk = max_pages_per_seq, max_seqs, prefill_chunk
        self.use_graphs = use_graphs and self.device.type == "cuda"
        self.prefill_buf = StepBuffers(prefill_chunk, 1, max_pages_per_seq, self.device)
        self.decode_bufs: dict[int, StepBuffers] = {}
        self.graphs: dict[int, tuple[torch.cuda.CUDAGraph, torch.Tensor]] = {}
        self.h2d_bytes = 0
        self.d2h_bytes = 0

    # ---- prefill ------------------------------------------------------------------------------------
    def prefill(self, seq: Sequence, tokens: list[int]) -> int:
        """Append ``tokens`` to ``seq`` in chunks; returns the greedy next token after the last."""
        nxt = -1
        for c0 in range(0, len(tokens), self.chunk):
            part = tokens[c0:c0 + self.chunk]
            start, n = seq.kv_len, len(part)
            self.table.reserve(seq, start + n)
            b = self.prefill_buf
            b.tokens[0][:n] = torch.tensor(part, dtype=torch.int32)
            b.positions[0][:n] = torch.arange(start, start + n, dtype=torch.int32)
            b.slots[0][:n] = torch.tensor(self.table.slots(seq, start, n), dtype=torch.int32)
            pt = b.page_table[0].view(1, self.max_pages)
            pt.zero_()
            pt[0, :len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
            b.seq_lens[0][0] = start + n
            b.q_start[0][0], b.q_start[0][1] = 0, n
            b.last_rows[0][0] = n - 1
            self.h2d_bytes += b.upload()
            batch = Batch(b.tokens[1][:n], b.positions[1][:n], b.slots[1][:n], b.page_table[1].view(1, self.max_pages),
                          b.seq_lens[1][:1], b.q_start[1][:2], n, True, b.last_rows[1][:1], fresh=start == 0)
            logits = self.engine.forward(batch)
            seq.tokens.extend(part)
            seq.kv_len = start + n
            if c0 + self.chunk >= len(tokens):
                nxt = int(self.engine.greedy(logits)[0].item())
                self.d2h_bytes += 4
        return nxt

    # ---- decode -------------------------------------------------------------------------------------
    def _decode_batch(self, b: StepBuffers, S: int) -> Batch:
        return Batch(b.tokens[1][:S], b.positions[1][:S], b.slots[1][:S], b.page_table[1].view(self.max_seqs_of(b), self.max_pages)[:S],
                     b.seq_lens[1][:S], b.q_start[1][:S + 1], 1, False, None)

    @staticmethod
    def max_seqs_of(b: StepBuffers) -> int:
        return b.max_seqs

    def decode(self, seqs: list[Sequence], last_tokens: list[int]) -> list[int]:
        """One greedy decode step for every sequence; returns the new tokens."""
        S = len(seqs)
        if S not in self.decode_bufs:
            self.decode_bufs[S] = StepBuffers(S, S, self.max_pages, self.device)
        b = self.decode_bufs[S]
        pt = b.page_table[0].view(S, self.max_pages)
        for i, (s, tok) in enumerate(zip(seqs, last_tokens)):
            self.table.reserve(s, s.kv_len + 1)
            b.tokens[0][i] = tok
            b.positions[0][i] = s.kv_len
            b.slots[0][i] = s.pages[s.kv_len // PAGE] * PAGE + s.kv_len % PAGE
            n = len(s.pages)
            if pt[i, n - 1] != s.pages[-1] or n == 1:
                pt[i, :n] = torch.tensor(s.pages, dtype=torch.int32)
            b.seq_lens[0][i] = s.kv_len + 1
            b.q_start[0][i] = i
        b.q_start[0][S] = S
        self.h2d_bytes += b.upload()
        if self.use_graphs:
            if S not in self.graphs:
                batch = self._decode_batch(b, S)
                for _ in range(2):                       # warm-up: kernel attributes, descriptor caches
                    self.engine.greedy(self.engine.forward(batch))
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g):
                    out = self.engine.greedy(self.engine.forward(batch))
                self.graphs[S] = (g, out)
                while len(self.graphs) > self.max_graphs:
                    old = next(iter(self.graphs))
                    del self.graphs[old]
                    self.decode_bufs.pop(old, None)
            g, out = self.graphs.pop(S)
            self.graphs[S] = (g, out)          # most recently used last
            if hasattr(self.engine, "mirror"):
                self.engine.mirror(self._decode_batch(b, S))
            if hasattr(self.engine, "take_replay"):
                self.engine.take_replay(S)
            elif hasattr(self.engine, "announce"):
                self.engine.announce(S, 1, for_replay=True)
            g.replay()
        else:
            out = self.engine.greedy(self.engine.forward(self._decode_batch(b, S)))
        new = out[:S].tolist()
        self.d2h_bytes += 4 * S
        for s, tok, nt in zip(seqs, last_tokens, new):
            s.tokens.append(tok)
            s.kv_len += 1
        return new
