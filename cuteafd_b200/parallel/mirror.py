"""One driver for a tensor-parallel attention group: rank 0 holds the scheduler (or the generator) and every other rank
repeats its engine calls.

A tensor-parallel engine (models/tp_gqa.py, models/tp_mla.py) wants the same batch on every rank: the collectives are
inside its kernels.  ``MirroredEngine`` wraps rank 0's engine: before a forward step it broadcasts the step's
description (a 16-word header, then the token ids, positions, KV slots, page table, lengths and row offsets as one int32
payload, device to device over NCCL on the compute stream) and then runs the step itself; page copies of the KV cache
(copy-on-write of shared prefix pages) are mirrored the same way.  ``follow`` is the other ranks' loop: receive, rebuild
the batch, run the same step on the local shard, until rank 0 says stop.  Rank 0 may replay CUDA graphs (the backend
calls ``mirror`` itself before a replay; a forward that is being captured sends nothing, since a capture runs nothing);
a follower keeps its own graph bank: a decode geometry it has run eagerly twice is captured right after the second
run and replayed from then on, its inputs arriving in one static buffer.

Counterpart: the reference's second coordinator GPU follows the first through its peer-split step protocol
(rust/crates/cuteafd-daemon/src/shared/peer_split/attention.rs); one scheduler, two GPUs' worth of heads.
"""
from __future__ import annotations

import torch
import torch.distributed as dist

OP_FORWARD, OP_COPY_PAGE, OP_STOP = 1, 2, 3
HEADER_WORDS = 16


class _MirroredKv:
    """The KV cache of rank 0 with its page copies repeated on the followers; everything else passes through."""

    def __init__(self, kv, owner: "MirroredEngine"):
        self._kv, self._owner = kv, owner

    def copy_page(self, src: int, dst: int) -> None:
        self._owner._send_header([OP_COPY_PAGE, int(src), int(dst)])
        self._kv.copy_page(src, dst)

    def __getattr__(self, name):
        return getattr(self._kv, name)


class MirroredEngine:
    """Rank 0's engine as the backends see it: ``forward`` (and KV page copies) happen on every rank of the group."""

    def __init__(self, inner, group=None):
        self.inner, self.group = inner, group or dist.group.WORLD
        self.src = dist.get_global_rank(self.group, 0) if self.group is not dist.group.WORLD else 0
        self.kv = _MirroredKv(inner.kv, self)
        self.mirrored_steps = 0

    # the MTP depth's own step and the host-resident embedding rows are not mirrored: the backends see neither
    HIDDEN = ("mtp_forward", "embed_rows")

    def __getattr__(self, name):                      # cfg, W, device, logits, next_tokens, greedy, launches, ...
        if name in MirroredEngine.HIDDEN or name in ("inner", "group"):
            raise AttributeError(name)
        return getattr(self.inner, name)

    def _send_header(self, words: list[int]) -> None:
        h = torch.tensor(words + [0] * (HEADER_WORDS - len(words)), dtype=torch.int64).to(self.inner.device)
        dist.broadcast(h, src=self.src, group=self.group)

    def mirror(self, b) -> None:
        """Send the step ``b`` describes to the followers (they run it as soon as it arrives)."""
        if getattr(b, "embeds", None) is not None:
            raise ValueError("media rows are not mirrored to a tensor-parallel group: text requests only")
        T, (S, max_pages) = b.tokens.shape[0], b.page_table.shape
        last = b.last_rows
        self._send_header([OP_FORWARD, T, S, max_pages, int(b.max_q_len), int(bool(b.prefill)), int(bool(getattr(b, "fresh", False))),
                           0 if last is None else 1, 0 if last is None else int(last.shape[0])])
        parts = [b.tokens, b.positions, b.slots, b.page_table.reshape(-1), b.seq_lens, b.q_start] + ([] if last is None else [last])
        payload = torch.cat([p.reshape(-1).to(torch.int32) for p in parts])
        dist.broadcast(payload, src=self.src, group=self.group)
        self.mirrored_steps += 1

    def forward(self, b):
        if not (self.inner.device.type == "cuda" and torch.cuda.is_current_stream_capturing()):
            self.mirror(b)
        return self.inner.forward(b)

    def take_replay(self, rows: int) -> None:         # the graph bank's hook before a replay: ``mirror`` was called with the batch
        return None

    def stop(self) -> None:
        self._send_header([OP_STOP])


class FollowerStats:
    def __init__(self) -> None:
        self.steps = self.replays = self.captures = 0


def follow(inner, group=None, on_step=None, graphs: bool = True, max_graphs: int = 32, stats: FollowerStats | None = None) -> int:
    """The loop of a rank that is not rank 0: repeat every mirrored call on the local shard.  Returns the number of
    forward steps it ran.  ``graphs``: decode steps of a geometry seen twice run from a CUDA graph of this rank's own
    (the step's description is received into one static buffer, so a graph's inputs never move)."""
    from ..models.gqa_moe import Batch
    group = group or dist.group.WORLD
    src = dist.get_global_rank(group, 0) if group is not dist.group.WORLD else 0
    dev, steps = inner.device, 0
    stats = stats or FollowerStats()
    graphs = graphs and dev.type == "cuda"
    static = torch.empty(1 << 16, dtype=torch.int32, device=dev)
    bank: dict[tuple, torch.cuda.CUDAGraph] = {}
    seen: dict[tuple, int] = {}
    while True:
        h = torch.zeros(HEADER_WORDS, dtype=torch.int64, device=dev)
        dist.broadcast(h, src=src, group=group)
        w = [int(v) for v in h.tolist()]
        if w[0] == OP_STOP:
            return steps
        if w[0] == OP_COPY_PAGE:
            inner.kv.copy_page(w[1], w[2])
            continue
        if w[0] != OP_FORWARD:
            raise RuntimeError(f"mirror: unknown message {w[:4]}")
        _, T, S, max_pages, max_q_len, prefill, fresh, has_last, n_last = w[:9]
        sizes = [T, T, T, S * max_pages, S, S + 1] + ([n_last] if has_last else [])
        n = sum(sizes)
        if n > static.numel():                       # a wider step than any before: the graphs' inputs lived in the old buffer
            static = torch.empty(2 * n, dtype=torch.int32, device=dev)
            bank.clear()
            seen.clear()
        payload = static[:n]
        dist.broadcast(payload, src=src, group=group)
        f = list(torch.split(payload, sizes))
        b = Batch(f[0], f[1], f[2], f[3].view(S, max_pages), f[4], f[5], max_q_len, bool(prefill), f[6] if has_last else None,
                  fresh=bool(fresh))
        key = tuple(w[1:9])
        with torch.no_grad():
            if key in bank:
                bank[key].replay()
                stats.replays += 1
            else:
                inner.forward(b)
                if graphs and not prefill:
                    seen[key] = seen.get(key, 0) + 1
                    if seen[key] == 2 and len(bank) < max_graphs:
                        # two eager runs have warmed this geometry up; record it now (a capture runs nothing, so the
                        # group's step count stays what rank 0 made it)
                        torch.cuda.synchronize(dev)
                        g = torch.cuda.CUDAGraph()
                        with torch.cuda.graph(g):
                            inner.forward(b)
                        bank[key] = g
                        stats.captures += 1
        steps += 1
        stats.steps = steps
        if on_step is not None:
            on_step(steps)
