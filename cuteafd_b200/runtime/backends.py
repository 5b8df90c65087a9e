"""Scheduler backends: the CUDA engine and the CPU oracle.

Both keep their KV bookkeeping in the same ``PagePool`` / ``SequenceTable`` / ``PrefixCache``
objects, so admission, prefix reuse, copy-on-write and eviction behave identically; only where
the KV bytes live differs (device page pools versus per-sequence oracle tensors).  The oracle
backend is what the scheduler, API and speculation tests run on, like the reference's scheduler
test backend and fake server (rust/crates/cuteafd-daemon/src/shared/qwen/scheduler.rs:1600-1670,
rust/crates/cuteafd-bench/examples/fake_server.rs:1-50).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from ..config import ModelConfig
from .native import make_pool
from .paged import PAGE, Sequence, SequenceTable
from .prefix_cache import PROMPT, TURN, PrefixCache


@dataclass
class _Handle:
    seq: Sequence
    kv: object = None            # oracle: KvState
    dead: bool = False
    media: object = None         # the request's media spans (rows whose embeddings come from a tower)


class OracleBackend:
    """CPU reference decoder behind the scheduler's Backend protocol."""

    def __init__(self, cfg: ModelConfig, params: dict[str, torch.Tensor], total_pages: int = 512, prefill_chunk: int = 64,
                 max_decode_rows: int = 64, fail_on_step: int | None = None, host_slots: int = 0):
        from ..ref.model import RefDecoder
        self.cfg, self.model = cfg, RefDecoder(cfg, params)
        self.vocab_size, self.prefill_chunk, self.max_decode_rows = cfg.vocab_size, prefill_chunk, max_decode_rows
        self.total_pages = total_pages
        self.pool = make_pool(total_pages)
        self.table = SequenceTable(self.pool)
        self.prefix = PrefixCache(self.pool, self.table, max_pages=total_pages // 2)
        self.tier = None
        if host_slots:                            # host tier on a virtual clock: the oracle's KV rides in the snapshot marks
            from .host_tier import HostTier
            from .hostcache import HostCache, StubCopyEngine
            self.tier = HostTier(self.prefix, self.pool, self.table, HostCache(StubCopyEngine(1 << 16), host_slots))
        self.steps = 0
        self.model.usage = {}                     # routed-token counters behind ``expert_usage``
        self.fail_on_step = fail_on_step          # host-side fault injection: the N-th verify raises
        self.quarantined: list[_Handle] = []
        self.has_mtp = cfg.mtp_layers > 0 and f"model.layers.{cfg.num_layers}.eh_proj.weight" in params
        self.last_mtp: list[int] | None = None
        if self.has_mtp:
            self.verify_select = self._verify_select     # selection next to the model, as on the GPU backend

    def expert_usage(self) -> dict:
        """Routed tokens per layer and expert since start, with the load imbalance (max / mean) per layer."""
        layers = {}
        for layer, c in sorted((self.model.usage or {}).items()):
            total = int(c.sum())
            layers[str(layer)] = {"tokens": c.tolist(), "total": total,
                                  "imbalance": round(float(c.max()) * c.numel() / total, 3) if total else None,
                                  "idle_experts": int((c == 0).sum())}
        return {"experts": self.cfg.num_experts, "top_k": self.cfg.top_k, "layers": layers}

    def _verify_select(self, handles: list[_Handle], rows: list[list[int]], params: list, positions: list[int]):
        """Forward, exact selection and the MTP depth on the same rows (the oracle of ``EngineBackend.verify_select``)."""
        from . import sampling
        self.steps += 1
        if self.fail_on_step is not None and self.steps == self.fail_on_step:
            raise RuntimeError("injected worker failure")
        toks, status, mtp, off = [], [], [], 0
        for h, r in zip(handles, rows):
            self.table.reserve(h.seq, h.seq.kv_len + len(r))
            start = h.seq.kv_len
            with torch.no_grad():
                hid = self.model.hidden_states(torch.tensor(r), h.kv)
                logits = self.model.head(hid)
                t, s = sampling.select_rows(logits, params[off:off + len(r)], positions[off:off + len(r)])
                nxt = torch.tensor([max(x, 0) for x in t])
                ml, _ = self.model.mtp_forward(0, hid, nxt, torch.arange(start, start + len(r)), h.kv)
            toks += t; status += s
            mtp += ml.argmax(-1).tolist()
            off += len(r)
            h.seq.tokens.extend(r)
            h.seq.kv_len += len(r)
        self.last_mtp = mtp
        return toks, status

    def open(self, tokens: list[int], cold: bool = False) -> tuple[_Handle, int]:
        from ..ref.model import KvState
        if cold:                                   # probe: compute the whole prompt, whatever the cache holds
            return _Handle(self.table.new(), KvState(self.cfg)), 0
        seq, m = self.prefix.admit(tokens)
        kv = KvState(self.cfg)
        got = self.tier.try_restore(tokens, m.length) if self.tier is not None else None
        if got is not None and got[2].mark is not None:
            self.table.free(seq)
            seq, length, hs = got
            kv.rows = [[r[0][:length].clone()] if r else [] for r in hs.mark.rows]
            return _Handle(seq, kv), length
        if got is not None:
            self.table.free(got[0])
        if m.length and m.snapshot is not None and m.snapshot.mark is not None:
            src = m.snapshot.mark
            kv.rows = [[r[0][:m.length].clone()] if r else [] for r in src.rows]
        elif m.length:
            # pages matched through the radix without a snapshot mark at that exact length:
            # find any snapshot covering the prefix and slice its state
            src = next((s.mark for s in self.prefix.snapshots.values()
                        if s.mark is not None and s.length >= m.length and s.tokens[:m.length] == tuple(tokens[:m.length])), None)
            if src is None:
                self.table.free(seq)
                seq, m.length = self.table.new(), 0
            else:
                kv.rows = [[r[0][:m.length].clone()] if r else [] for r in src.rows]
        return _Handle(seq, kv), m.length

    def prefill(self, h: _Handle, tokens: list[int], last: bool):
        from ..media.processor import overrides_for
        self.table.reserve(h.seq, h.seq.kv_len + len(tokens))
        start = h.seq.kv_len
        ov = overrides_for(getattr(h, "media", None), start, len(tokens))
        with torch.no_grad():
            hid = self.model.hidden_states(torch.tensor(tokens), h.kv, ov)
            if self.has_mtp:                 # the MTP depth's K/V for the prompt (see EngineBackend.prefill)
                self.model.mtp_forward(0, hid, torch.tensor(tokens[1:] + tokens[-1:]), torch.arange(start, start + len(tokens)), h.kv)
        h.seq.tokens.extend(tokens)
        h.seq.kv_len += len(tokens)
        return self.model.head(hid[-1:]) if last else None

    def prefill_packed(self, items: list) -> list:
        """[(handle, tokens, last)] -> logits of the last row for the items that end their prompt, else None."""
        return [self.prefill(h, toks, last) for h, toks, last in items]

    def verify(self, handles: list[_Handle], rows: list[list[int]]) -> torch.Tensor:
        self.steps += 1
        if self.fail_on_step is not None and self.steps == self.fail_on_step:
            raise RuntimeError("injected worker failure")
        out = []
        for h, r in zip(handles, rows):
            self.table.reserve(h.seq, h.seq.kv_len + len(r))
            with torch.no_grad():
                out.append(self.model.forward(torch.tensor(r), h.kv))
            h.seq.tokens.extend(r)
            h.seq.kv_len += len(r)
        return torch.cat(out, 0)

    def commit(self, h: _Handle, keep_tokens: int) -> None:
        if keep_tokens < h.seq.kv_len:
            self.table.truncate(h.seq, keep_tokens)
            h.kv.truncate(keep_tokens)

    def capture(self, h: _Handle, kind: str) -> None:
        import copy
        self.prefix.capture(h.seq, PROMPT if kind == "prompt" else TURN, mark=copy.deepcopy(h.kv))

    def release(self, h: _Handle) -> None:
        if not h.dead:
            self.table.free(h.seq)
            h.dead = True

    def quarantine(self, h: _Handle) -> None:
        h.dead = True
        self.quarantined.append(h)            # pages stay allocated: never handed to another request

    def state_hash(self, h: _Handle) -> str:
        """Probe ``record_state``: hash of the sequence's cached rows, every layer, in position order."""
        import hashlib
        d = hashlib.blake2b(digest_size=16)
        for rows in h.kv.rows:
            for r in rows:
                d.update(r.detach().float().contiguous().numpy().tobytes())
        return d.hexdigest()

    def pages_of(self, h: _Handle) -> int:
        return len(h.seq.pages)


def pt_dev(b, max_pages: int) -> torch.Tensor:
    """Device page table of a ``StepBuffers`` as [max_seqs, max_pages]."""
    return b.page_table[1].view(b.max_seqs, max_pages)


class EngineBackend:
    """The CUDA engine (single GPU or the attention rank of an AFD group)."""

    def __init__(self, engine, num_pages: int, max_pages_per_seq: int, prefill_chunk: int = 2048, max_decode_rows: int = 64,
                 use_graphs: bool = True, host_cache_bytes: int = 0, host_embedding=None):
        from .generate import Generator, StepBuffers
        self.engine = engine
        self.cfg = engine.cfg
        self.vocab_size = self.cfg.vocab_size
        self.prefill_chunk, self.max_decode_rows = prefill_chunk, max_decode_rows
        self.total_pages = num_pages
        self.pool = make_pool(num_pages)
        self.gen = Generator(engine, self.pool, max_pages_per_seq, max_decode_rows, prefill_chunk, use_graphs)
        self.table = self.gen.table
        self.prefix = PrefixCache(self.pool, self.table, max_pages=num_pages // 2)
        self.tier = None
        if host_cache_bytes > 0 and engine.device.type == "cuda":
            # pinned-host tier behind the device cache: evicted snapshots are copied out on a side stream and come
            # back through the same engine when a later request asks for their prefix
            from .host_tier import HostTier
            from .hostcache import CudaCopyEngine, HostCache
            kv = engine.kv if hasattr(engine, "kv") else engine.inner.kv
            pools = list(getattr(kv, "k", [])) + list(getattr(kv, "v", [])) + list(getattr(kv, "c", [])) + list(getattr(kv, "idx", []))
            slots = int(host_cache_bytes // max(1, kv.bytes_per_page()))
            if slots >= 8:
                self.tier = HostTier(self.prefix, self.pool, self.table, HostCache(CudaCopyEngine(pools, slots), slots))
        # Host-resident embedding table (``loader/mapped_table.py``): every step's rows are gathered from the memory-mapped
        # checkpoint file by the table's thread pool into pinned memory and copied into the engine's fixed staging buffer
        # before the step is launched; the next prompt chunk's rows are prefetched while the current one computes.  The
        # reference keeps token embeddings (and DeepSeek's per-layer tables) on the host the same way
        # (run.sh --embedding-placement host; rust/crates/cuteafd-loader/src/formats/mapped_table.rs).
        self.host_embed = host_embedding
        if host_embedding is not None:
            rows = max(self.gen.prefill_buf.tokens[0].numel(), max_decode_rows * 8)
            engine.embed_rows = torch.zeros(rows, self.cfg.hidden, dtype=torch.bfloat16, device=engine.device)
            self._embed_stage = torch.zeros(rows, self.cfg.hidden, dtype=torch.bfloat16).pin_memory()
        self.max_pages = max_pages_per_seq
        # longest sequence one page-table row can describe (speculative rows of the last step included)
        self.max_context_tokens = max(PAGE, (max_pages_per_seq - 1) * PAGE)
        self.bufs = StepBuffers(max_decode_rows * 8, max_decode_rows, max_pages_per_seq, engine.device)
        self.quarantined: list[_Handle] = []
        self._sel = None
        self._last_batch = None
        self.last_mtp: list[int] | None = None
        # Decode graph bank: one CUDA graph per exact step geometry (sequences, rows, longest row run).  A geometry is
        # captured once it has been seen ``graph_after`` times (or named by a prewarm list), replayed from then on, and
        # dropped least recently used first beyond ``max_graphs``; a step never waits for a capture it does not need
        # (the eager path serves it).  Counterpart: rust/crates/cuteafd-daemon/src/shared/decode_graph/bank.rs.
        self.use_graphs = use_graphs
        self.max_graphs, self.graph_after = 32, 2
        self.graphs: dict[tuple[int, int, int], tuple] = {}
        self.geometry_seen: dict[tuple[int, int, int], int] = {}
        self.graph_stats = {"replays": 0, "eager": 0, "captures": 0, "evictions": 0, "refused": 0}
        # Byte-measured graph arena: every capture is charged the device memory it made the allocator reserve (the
        # graph's private pool), the bank stays under ``graph_budget_bytes`` by dropping least recently used graphs, and a
        # capture that would not fit even then is refused (that geometry stays on the eager path).  The measured base
        # (sum) and extra (largest single capture: the tail one more capture may need) go into the prewarm file, where
        # the planner reads its graph reserve from.  Counterpart: rust/crates/cuteafd-loader/src/placement/graph_reserve.rs
        # (trace-derived base + extra per rank).
        self.graph_bytes: dict[tuple[int, int, int], int] = {}
        self.graph_budget_bytes = 0                       # 0 = no byte budget (the count limit still applies)
        inner = getattr(engine, "inner", engine)
        self.has_mtp = (bool(getattr(getattr(inner, "W", None), "mtp", None)) and hasattr(engine, "mtp_forward")
                        and host_embedding is None)      # the MTP depth embeds the selected tokens on the device

    def _stage_embeddings(self, host_tokens: torch.Tensor, lookahead=None) -> None:
        """Rows of the host embedding table for the step whose token ids were just staged (no-op with the table on the
        GPU); ``lookahead``: ids a later step will need (the next chunk of the prompt)."""
        if self.host_embed is None:
            return
        n = host_tokens.numel()
        sent = getattr(self, "_embed_sent", None)
        if sent is not None:
            sent.synchronize()              # the previous step's copy has read the staging rows
        self.host_embed.gather(host_tokens.numpy(), out=self._embed_stage[:n])
        self.engine.embed_rows[:n].copy_(self._embed_stage[:n], non_blocking=True)
        if self._embed_stage.is_pinned():
            if sent is None:
                sent = self._embed_sent = torch.cuda.Event()
            sent.record()
        if lookahead:
            self.host_embed.prefetch(lookahead)

    def _copy_page(self, src: int, dst: int) -> None:
        kv = self.engine.kv if hasattr(self.engine, "kv") else self.engine.inner.kv
        kv.copy_page(src, dst)

    def expert_usage(self) -> dict:
        """A sample, not a total: the routed-token counts the planner kernel left for the last MoE layer of the last
        step (the exchange keeps one counter vector and every layer overwrites it; accumulating on the device would add
        a launch per layer to every decode step)."""
        moe = getattr(self.engine, "moe", None)
        c = getattr(moe, "expert_count", None)
        if c is None:
            return {}
        try:
            t = c.detach().to("cpu", torch.int64)
        except RuntimeError:
            return {}
        total = int(t.sum())
        return {"experts": int(t.numel()), "top_k": self.cfg.top_k, "sample": "last MoE layer of the last step",
                "tokens": t.tolist(), "total": total,
                "imbalance": round(float(t.max()) * t.numel() / total, 3) if total else None}

    def open(self, tokens: list[int], cold: bool = False) -> tuple[_Handle, int]:
        if cold:                                   # probe: compute the whole prompt, whatever the cache holds
            return _Handle(self.table.new()), 0
        seq, m = self.prefix.admit(tokens)
        got = self.tier.try_restore(tokens, m.length) if self.tier is not None else None
        if got is not None:
            self.table.free(seq)
            return _Handle(got[0]), got[1]
        return _Handle(seq), m.length

    def prefill(self, h: _Handle, tokens: list[int], last: bool):
        from ..models.gqa_moe import Batch
        seq = h.seq
        start, n = seq.kv_len, len(tokens)
        self.table.reserve(seq, start + n, copy_page=self._copy_page)
        b = self.gen.prefill_buf
        # ids above the vocabulary mark media rows (their embeddings come from the request's spans); the embedding
        # kernel still needs a valid id there
        V = self.vocab_size
        ov = None
        if any(t >= V for t in tokens):
            from ..media.processor import overrides_for
            ov = overrides_for(getattr(h, "media", None), start, n)
            if ov is None or len(ov[0]) != sum(t >= V for t in tokens):
                raise ValueError("media rows in the prompt without their embeddings")
        b.tokens[0][:n] = torch.tensor([t if t < V else 0 for t in tokens] if ov is not None else tokens, dtype=torch.int32)
        b.positions[0][:n] = torch.arange(start, start + n, dtype=torch.int32)
        b.slots[0][:n] = torch.tensor(self.table.slots(seq, start, n), dtype=torch.int32)
        pt = b.page_table[0].view(1, self.max_pages)
        pt.zero_()
        pt[0, :len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
        b.seq_lens[0][0] = start + n
        b.q_start[0][0], b.q_start[0][1] = 0, n
        b.last_rows[0][0] = n - 1
        b.upload()
        self._stage_embeddings(b.tokens[0][:n])
        batch = Batch(b.tokens[1][:n], b.positions[1][:n], b.slots[1][:n], b.page_table[1].view(1, self.max_pages),
                      b.seq_lens[1][:1], b.q_start[1][:2], n, True, b.last_rows[1][:1], fresh=start == 0)
        if ov is not None:
            dev = self.engine.device
            batch.embeds = (torch.tensor(ov[0], dtype=torch.long).to(dev), ov[1].to(dev, torch.bfloat16))
        logits = self.engine.forward(batch)
        if self.has_mtp:
            # fill the MTP depth's K/V for the prompt: position t pairs with prompt token t+1 (the chunk's last row
            # repeats its own token: its true successor is not known yet; it only colours one draft)
            nxt = torch.tensor(tokens[1:] + tokens[-1:], dtype=torch.int32).to(self.engine.device, non_blocking=True)
            self.engine.mtp_forward(0, batch, nxt)
        seq.tokens.extend(tokens)
        seq.kv_len = start + n
        return logits[:1].float().cpu() if last else None

    def prefill_packed(self, items: list) -> list:
        """Chunks of several prompts in one forward step: [(handle, tokens, last)] -> per item the fp32 logits of its
        last row when ``last`` (on the host), else None.  Media rows and the MTP fill work as in ``prefill``."""
        from ..models.gqa_moe import Batch
        from ..media.processor import overrides_for
        from .generate import StepBuffers
        S, T = len(items), sum(len(t) for _, t, _ in items)
        if getattr(self, "_pack_bufs", None) is None:
            self._pack_bufs = StepBuffers(self.prefill_chunk, 16, self.max_pages, self.engine.device)
        b = self._pack_bufs
        assert S <= b.max_seqs and T <= b.max_tokens
        V = self.vocab_size
        pt = b.page_table[0].view(b.max_seqs, self.max_pages)
        o, rows, vals, nxt = 0, [], [], []
        for i, (h, toks, _) in enumerate(items):
            seq = h.seq
            start, n = seq.kv_len, len(toks)
            self.table.reserve(seq, start + n, copy_page=self._copy_page)
            if any(t >= V for t in toks):
                ov = overrides_for(getattr(h, "media", None), start, n)
                if ov is None or len(ov[0]) != sum(t >= V for t in toks):
                    raise ValueError("media rows in the prompt without their embeddings")
                rows += [o + r for r in ov[0]]
                vals.append(ov[1])
            b.tokens[0][o:o + n] = torch.tensor([t if t < V else 0 for t in toks], dtype=torch.int32)
            b.positions[0][o:o + n] = torch.arange(start, start + n, dtype=torch.int32)
            b.slots[0][o:o + n] = torch.tensor(self.table.slots(seq, start, n), dtype=torch.int32)
            pt[i].zero_()
            pt[i, :len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
            b.seq_lens[0][i] = start + n
            b.q_start[0][i] = o
            b.last_rows[0][i] = o + n - 1
            nxt += toks[1:] + toks[-1:]
            o += n
        b.q_start[0][S] = T
        b.upload()
        self._stage_embeddings(b.tokens[0][:T])
        batch = Batch(b.tokens[1][:T], b.positions[1][:T], b.slots[1][:T], pt_dev(b, self.max_pages)[:S], b.seq_lens[1][:S],
                      b.q_start[1][:S + 1], max(len(t) for _, t, _ in items), True, b.last_rows[1][:S], fresh=False)
        if rows:
            dev = self.engine.device
            batch.embeds = (torch.tensor(rows, dtype=torch.long).to(dev), torch.cat(vals).to(dev, torch.bfloat16))
        logits = self.engine.forward(batch)
        if self.has_mtp:
            self.engine.mtp_forward(0, batch, torch.tensor([t if t < V else 0 for t in nxt], dtype=torch.int32).to(self.engine.device))
        host = logits[:S].float().cpu() if any(last for _, _, last in items) else None
        out = []
        for i, (h, toks, last) in enumerate(items):
            h.seq.tokens.extend(toks)
            h.seq.kv_len += len(toks)
            out.append(host[i:i + 1] if last else None)
        return out

    # ---- decode graph bank ------------------------------------------------------------------------------
    def _step_batch(self, key: tuple[int, int, int]):
        from ..models.gqa_moe import Batch
        S, T, mq = key
        b = self.bufs
        return Batch(b.tokens[1][:T], b.positions[1][:T], b.slots[1][:T], b.page_table[1].view(b.max_seqs, self.max_pages)[:S],
                     b.seq_lens[1][:S], b.q_start[1][:S + 1], mq, False, None)

    def _capture(self, key: tuple[int, int, int], batch) -> None:
        """The step's inputs are already in the static buffers.  Kernels run during the warm-up write the same K/V the
        replay writes again, so capturing in the middle of serving is harmless."""
        for _ in range(2):
            self.engine.forward(batch)
        torch.cuda.synchronize()
        if self.graph_budget_bytes:
            guess = max(self.graph_bytes.values(), default=0)          # what one more capture is likely to take
            while self.graphs and self.graph_bytes_total() + guess > self.graph_budget_bytes:
                self._evict_oldest()
            if self.graph_bytes_total() + guess > self.graph_budget_bytes:
                self.graph_stats["refused"] += 1
                return
        before = torch.cuda.memory_reserved(self.engine.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            out = self.engine.forward(batch)
        torch.cuda.synchronize()
        self.graphs[key] = (g, out)
        self.graph_bytes[key] = max(0, torch.cuda.memory_reserved(self.engine.device) - before)
        self.graph_stats["captures"] += 1
        while len(self.graphs) > self.max_graphs or (self.graph_budget_bytes and len(self.graphs) > 1
                                                     and self.graph_bytes_total() > self.graph_budget_bytes):
            self._evict_oldest()

    def _evict_oldest(self) -> None:
        old = next(iter(self.graphs))
        del self.graphs[old]
        self.graph_bytes.pop(old, None)
        self.graph_stats["evictions"] += 1

    def graph_bytes_total(self) -> int:
        return sum(self.graph_bytes.get(k, 0) for k in self.graphs)

    def graph_reserve(self) -> dict:
        """Measured arena of the graphs held now: base = their sum, extra = the largest single capture."""
        return {"reserve_base_bytes": self.graph_bytes_total(), "reserve_extra_bytes": max(self.graph_bytes.values(), default=0),
                "graphs": len(self.graphs), "budget_bytes": self.graph_budget_bytes}

    def _run_step(self, key: tuple[int, int, int], batch) -> torch.Tensor:
        seen = self.geometry_seen[key] = self.geometry_seen.get(key, 0) + 1
        if self.use_graphs and key not in self.graphs and seen >= self.graph_after:
            self._capture(key, batch)
        if self.use_graphs and key in self.graphs:
            g, out = self.graphs.pop(key)
            self.graphs[key] = (g, out)                       # most recently used last
            if hasattr(self.engine, "mirror"):
                self.engine.mirror(batch)                     # tensor-parallel followers get the step a replay runs
            if hasattr(self.engine, "take_replay"):
                self.engine.take_replay(key[1])
            elif hasattr(self.engine, "announce"):
                self.engine.announce(key[1], 1, for_replay=True)
            g.replay()
            self.graph_stats["replays"] += 1
            return out
        self.graph_stats["eager"] += 1
        return self.engine.forward(batch)

    def prewarm(self, keys: list) -> int:
        """Capture the listed geometries before traffic arrives ([sequences, rows, longest run] triples, e.g. the list a
        previous run saved with ``save_prewarm``).  The capture runs on a dummy step: no K/V slot is written (slot -1),
        every table entry is the zero page.  Returns the number of graphs captured."""
        if not self.use_graphs:
            return 0
        b = self.bufs
        n = 0
        for key in keys:
            S, T, mq = (int(v) for v in key)
            if (S, T, mq) in self.graphs or S < 1 or S > b.max_seqs or T < S or T > b.max_tokens or mq * S < T:
                continue
            b.tokens[0][:T] = 0
            b.positions[0][:T] = 0
            b.slots[0][:T] = -1
            b.page_table[0].zero_()
            b.seq_lens[0][:S] = mq
            per, extra = divmod(T, S)
            starts = [0]
            for i in range(S):
                starts.append(starts[-1] + per + (1 if i < extra else 0))
            b.q_start[0][:S + 1] = torch.tensor(starts, dtype=torch.int32)
            b.upload()
            self._stage_embeddings(b.tokens[0][:T])
            self._capture((S, T, mq), self._step_batch((S, T, mq)))
            n += 1
        return n

    def save_prewarm(self, path: str, top: int = 16) -> list:
        """Write the most frequent step geometries of this run as a prewarm list (JSON)."""
        import json
        keys = [list(k) for k, _ in sorted(self.geometry_seen.items(), key=lambda kv: -kv[1])[:top]]
        with open(path, "w") as f:
            json.dump({"geometries": keys, "seen": {",".join(map(str, k)): v for k, v in self.geometry_seen.items()},
                       "graph_bytes": {",".join(map(str, k)): v for k, v in self.graph_bytes.items()}, **self.graph_reserve()}, f)
        return keys

    def _verify_device(self, handles: list[_Handle], rows: list[list[int]]) -> torch.Tensor:
        from ..models.gqa_moe import Batch
        S = len(handles)
        T = sum(len(r) for r in rows)
        b = self.bufs
        pt = b.page_table[0].view(b.max_seqs, self.max_pages)
        o = 0
        for i, (h, r) in enumerate(zip(handles, rows)):
            seq = h.seq
            self.table.reserve(seq, seq.kv_len + len(r), copy_page=self._copy_page)
            n = len(r)
            b.tokens[0][o:o + n] = torch.tensor(r, dtype=torch.int32)
            b.positions[0][o:o + n] = torch.arange(seq.kv_len, seq.kv_len + n, dtype=torch.int32)
            b.slots[0][o:o + n] = torch.tensor(self.table.slots(seq, seq.kv_len, n), dtype=torch.int32)
            pt[i].zero_()
            pt[i, :len(seq.pages)] = torch.tensor(seq.pages, dtype=torch.int32)
            b.seq_lens[0][i] = seq.kv_len + n
            b.q_start[0][i] = o
            o += n
        b.q_start[0][S] = T
        b.upload()
        self._stage_embeddings(b.tokens[0][:T])
        key = (S, T, max(len(r) for r in rows))
        batch = self._step_batch(key)
        logits = self._run_step(key, batch)
        for h, r in zip(handles, rows):
            h.seq.tokens.extend(r)
            h.seq.kv_len += len(r)
        self._last_batch = batch
        return logits[:T]

    def verify(self, handles: list[_Handle], rows: list[list[int]]) -> torch.Tensor:
        from ..ops import kernels as K
        out = self._verify_device(handles, rows).float().cpu()
        st = K.read_status()
        if st:
            raise RuntimeError(f"a bounded device wait ran out (status {st})")
        return out

    def verify_select(self, handles: list[_Handle], rows: list[list[int]], params: list, positions: list[int]) -> tuple[list[int], list[int]]:
        """Forward + exact target sampling on the GPU: one 64-byte record per row goes up, 8 bytes per row
        come back (token, row status) instead of a full-vocabulary logit row."""
        from ..ops import kernels as K
        logits = self._verify_device(handles, rows)
        T = logits.shape[0]
        rec = K.pack_sample_rows(params, positions)
        if self._sel is None or self._sel[0].shape[0] < T:
            n = max(T, self.bufs.max_tokens)
            self._sel = (torch.empty(n, 64, dtype=torch.uint8, device=self.engine.device),
                         torch.zeros(3, n, dtype=torch.int32, device=self.engine.device),
                         torch.empty(n, 64, dtype=torch.uint8).pin_memory())
        dev_rec, dev_out, host_rec = self._sel
        if getattr(self, "_rec_sent", None) is None:
            self._rec_sent = torch.cuda.Event()
        else:
            self._rec_sent.synchronize()    # the previous step's copy has read the staging records
        host_rec[:T].copy_(rec)
        dev_rec[:T].copy_(host_rec[:T], non_blocking=True)
        self._rec_sent.record()
        K.sample_rows(logits, dev_rec[:T], dev_out[0, :T], dev_out[1, :T])
        self.last_mtp = None
        if self.has_mtp:
            # MTP depth on the same rows: (final hidden of row t, token selected for row t) -> draft of the token after.
            # Rows past a sequence's accepted prefix compute drafts nobody reads and K/V that the commit truncates.
            nxt = torch.clamp_min(dev_out[0, :T], 0)
            mtp_logits = self.engine.mtp_forward(0, self._last_batch, nxt)
            n = mtp_logits.shape[0]
            K.argmax(mtp_logits, out=dev_out[2, :n])
        out = dev_out[:, :T].cpu()
        if self.has_mtp:
            self.last_mtp = out[2].tolist()
        st = K.read_status()
        if st:
            raise RuntimeError(f"a bounded device wait ran out (status {st})")
        return out[0].tolist(), out[1].tolist()

    def commit(self, h: _Handle, keep_tokens: int) -> None:
        if keep_tokens < h.seq.kv_len:
            self.table.truncate(h.seq, keep_tokens)

    def capture(self, h: _Handle, kind: str) -> None:
        self.prefix.capture(h.seq, PROMPT if kind == "prompt" else TURN)

    def release(self, h: _Handle) -> None:
        if not h.dead:
            self.table.free(h.seq)
            h.dead = True

    def quarantine(self, h: _Handle) -> None:
        h.dead = True
        self.quarantined.append(h)

    def state_hash(self, h: _Handle) -> str:
        """Probe ``record_state``: hash of the bytes the sequence's positions [0, kv_len) hold in every paged pool
        (K / V pages, latent records, index vectors), every layer, in position order.  Synchronous: the pages are copied
        to the host.  Two sequences with the same tokens hash equal whatever pages they sit in
        (rust/crates/cuteafd-api/src/openai/probe.rs:94-96)."""
        import hashlib
        kv = self.engine.kv if hasattr(self.engine, "kv") else self.engine.inner.kv
        seq, d = h.seq, hashlib.blake2b(digest_size=16)
        n = seq.kv_len
        if n == 0:
            return d.hexdigest()
        pages = torch.tensor(seq.pages[: (n + PAGE - 1) // PAGE], dtype=torch.long, device=self.engine.device)
        tail = n - (len(pages) - 1) * PAGE
        for name in ("k", "v", "c", "idx"):
            for pool in getattr(kv, name, []) or []:
                got = pool.index_select(0, pages)                    # [pages, ..., 64 positions, ...]
                ax = 2 if name in ("k", "v") else 1                  # K / V pages are [page, head, position, dim]
                last = got[-1:].narrow(ax, 0, tail)
                for part in (got[:-1], last):
                    if part.numel():
                        d.update(part.contiguous().view(torch.uint8).cpu().numpy().tobytes())
        return d.hexdigest()

    def pages_of(self, h: _Handle) -> int:
        return len(h.seq.pages)
