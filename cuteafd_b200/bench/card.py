"""Benchmark card: 8K cold prefill (tok/s, TTFT) and aggregate decode tok/s at several concurrencies.

Same phases as the reference's release-smoke card (rust/crates/cuteafd-bench/src/baseline.rs:1-25:
C1 decode, warmed C4/8/16 sweep with a distinct prompt per stream, cold exactly-8192-token
prefill with TTFT), widened to concurrency 32 and run in-process on synthetic token ids.

Two timings per decode level:
  * device: a CUDA graph holding one full step (forward, greedy select, device-side advance of
    token / position / KV slot) replayed K times between two CUDA events; no host work inside.
  * end to end: ``Generator.decode`` K times; every step copies its inputs from pinned host memory
    to the device and reads the selected tokens back.
"""
from __future__ import annotations

import time
from dataclasses import dataclass, field

import torch

from ..models.gqa_moe import Batch
from ..ops import kernels as K
from ..runtime.generate import Generator, StepBuffers
from ..runtime.paged import PAGE


@dataclass
class DecodeResult:
    concurrency: int
    steps: int
    ms_per_step: float
    tok_s: float
    e2e_ms_per_step: float
    e2e_tok_s: float
    launches_per_step: int
    h2d_bytes_per_step: int
    d2h_bytes_per_step: int


@dataclass
class CardResult:
    prefill_tok_s: float = 0.0
    ttft_s: float = 0.0
    prefill_ms: list[float] = field(default_factory=list)
    decode: dict[int, DecodeResult] = field(default_factory=dict)


def _event_ms(fn) -> float:
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    torch.cuda.synchronize()
    a.record()
    fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b)


def device_decode_loop(gen: Generator, seqs, last_tokens: list[int], steps: int, warmup: int, sync=None) -> tuple[float, int]:
    """K graph replays of (forward + greedy + advance) with inputs resident on the device.
    Returns (milliseconds for ``steps`` steps, kernel launches per step)."""
    eng = gen.engine
    S = len(seqs)
    b = StepBuffers(S, S, gen.max_pages, gen.device)
    pt = b.page_table[0].view(S, gen.max_pages)
    for i, (s, tok) in enumerate(zip(seqs, last_tokens)):
        gen.table.reserve(s, s.kv_len + warmup + steps + 4)
        b.tokens[0][i] = tok
        b.positions[0][i] = s.kv_len
        b.slots[0][i] = s.pages[s.kv_len // PAGE] * PAGE + s.kv_len % PAGE
        pt[i, :len(s.pages)] = torch.tensor(s.pages, dtype=torch.int32)
        b.seq_lens[0][i] = s.kv_len + 1
        b.q_start[0][i] = i
    b.q_start[0][S] = S
    b.upload()
    batch = Batch(b.tokens[1][:S], b.positions[1][:S], b.slots[1][:S], b.page_table[1].view(S, gen.max_pages),
                  b.seq_lens[1][:S], b.q_start[1][:S + 1], 1, False, None)

    def step():
        if hasattr(eng, "decode_step"):          # forward + selection + device-side advance, one launch where the engine fuses it
            eng.decode_step(batch, advance=True)
            return
        out = eng.greedy(eng.forward(batch))
        K.decode_advance(batch.tokens, out, batch.positions, batch.seq_lens, batch.slots, batch.page_table)

    l0 = eng.launches
    step()                                   # eager once: attribute setup, descriptor caches, scratch
    launches = eng.launches - l0 + (0 if hasattr(eng, "decode_step") else 1)
    torch.cuda.synchronize()
    if gen.use_graphs:
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            step()
        run = g.replay
    else:
        run = step
    announce = getattr(eng, "announce", None) if gen.use_graphs else None
    if announce and warmup > 1:
        announce(S, warmup - 1, for_replay=True)
    for _ in range(max(0, warmup - 1)):
        run()
    if sync is not None:
        sync()
    if announce:
        announce(S, steps, timed=True, for_replay=True)
    elif hasattr(eng, "announce"):
        eng.announce(S, steps, timed=True)
    ms = _event_ms(lambda: [run() for _ in range(steps)])
    if hasattr(eng, "collect_max"):
        ms = eng.collect_max(ms)                 # max over ranks (expert ranks time the same steps)
    assert K.read_status() == 0, "a bounded wait ran out during the timed region"
    for s in seqs:                           # account for the tokens the device loop appended
        s.kv_len += warmup + steps
    return ms, launches


def e2e_decode_loop(gen: Generator, seqs, last_tokens: list[int], steps: int, warmup: int, sync=None) -> tuple[float, int, int]:
    toks = list(last_tokens)
    for _ in range(warmup):
        toks = gen.decode(seqs, toks)
    h0, d0 = gen.h2d_bytes, gen.d2h_bytes
    if sync is not None:
        sync()
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    for _ in range(steps):
        toks = gen.decode(seqs, toks)
    torch.cuda.synchronize()
    ms = (time.perf_counter() - t0) * 1e3
    return ms, (gen.h2d_bytes - h0) // steps, (gen.d2h_bytes - d0) // steps


def run_card(gen: Generator, prompts: list[list[int]], levels: tuple[int, ...], steps: int, warmup: int,
             sync=None, log=print, replica: int = 0, n_replicas: int = 1) -> CardResult:
    """``prompts``: one distinct prompt per stream of the widest level.

    With ``n_replicas`` data-parallel attention replicas every replica runs this same script: prompt / stream i belongs
    to replica i % n_replicas, replica 0 announces each round's token counts for everybody, and a replica without work
    in a round waits for the round to close.  Decode throughput counts the streams of all replicas over the slowest
    rank's device time; prefill throughput counts the prompts that were prefilled side by side."""
    res = CardResult()
    table = gen.table
    eng = gen.engine
    A, a = n_replicas, replica
    dp = A > 1

    def peers(counts_of) -> None:
        if dp and a == 0:
            eng.peer_counts = [counts_of(j) for j in range(1, A)]

    def close(active: bool) -> None:
        if dp:
            eng.end_round(active)

    # ---- cold 8K prefill + TTFT: one untimed warm prompt, then every stream's prompt timed ----------
    peers(lambda j: len(prompts[0]))
    warm = table.new()
    gen.prefill(warm, prompts[0])
    table.free(warm)
    torch.cuda.synchronize()
    close(True)
    base: dict[int, object] = {}
    first: dict[int, int] = {}
    rounds = -(-len(prompts) // A)
    side_by_side = []
    for r in range(rounds):
        idx = r * A + a
        active = idx < len(prompts)
        peers(lambda j: len(prompts[r * A + j]) if r * A + j < len(prompts) else 0)
        if active:
            s = table.new()
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            nxt = gen.prefill(s, prompts[idx])              # returns after the first token reached the host
            dt = time.perf_counter() - t0
            res.prefill_ms.append(dt * 1e3)
            base[idx], first[idx] = s, nxt
            side_by_side.append(min(A, len(prompts) - r * A))
        close(active)
    res.ttft_s = sorted(res.prefill_ms)[len(res.prefill_ms) // 2] / 1e3
    res.prefill_tok_s = len(prompts[0]) * (sorted(side_by_side)[len(side_by_side) // 2]) / res.ttft_s
    log(f"prefill: {res.prefill_tok_s:.0f} tok/s, TTFT {res.ttft_s*1e3:.1f} ms (median of {len(res.prefill_ms)}"
        + (f", {A} prompts side by side" if dp else "") + ")")
    # ---- decode levels --------------------------------------------------------------------------------
    for c in levels:
        mine = [i for i in range(c) if i % A == a]
        peers(lambda j: len([i for i in range(c) if i % A == j]))
        ms, launches = 0.0, 0
        if mine:
            seqs = [table.fork(base[i]) for i in mine]
            ms, launches = device_decode_loop(gen, seqs, [first[i] for i in mine], steps, warmup, sync)
            for s in seqs:
                table.free(s)
        close(bool(mine))
        e_ms, h2d, d2h = 0.0, 0, 0
        if mine:
            seqs = [table.fork(base[i]) for i in mine]
            e_ms, h2d, d2h = e2e_decode_loop(gen, seqs, [first[i] for i in mine], steps, warmup, sync)
            for s in seqs:
                table.free(s)
        close(bool(mine))
        if not mine:
            continue
        r = DecodeResult(c, steps, ms / steps, c * steps / (ms / 1e3), e_ms / steps, c * steps / (e_ms / 1e3),
                         launches, h2d, d2h)
        res.decode[c] = r
        log(f"decode C{c}: device {r.ms_per_step:.3f} ms/step {r.tok_s:.1f} tok/s | e2e {r.e2e_ms_per_step:.3f} ms/step "
            f"{r.e2e_tok_s:.1f} tok/s | {launches} launches/step")
    for s in base.values():
        table.free(s)
    return res
