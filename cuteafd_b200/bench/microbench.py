"""Kernel microbenchmarks with roofline fractions (CUDA-event timing, L2 flushed between runs).

    python -m cuteafd_b200.bench.microbench gemm --tokens 8192 --features 5120 --k 2048
    python -m cuteafd_b200.bench.microbench attn-prefill --len 8192
    python -m cuteafd_b200.bench.microbench attn-decode --seqs 32 --len 8192
    python -m cuteafd_b200.bench.microbench mla --seqs 8 --len 8192 --qlen 1 --heads 128 [--topk 2048]
    python -m cuteafd_b200.bench.microbench w4 --tokens 8 --features 7168 --k 2048 --fmt nvfp4
    python -m cuteafd_b200.bench.microbench sampler --rows 32 --vocab 151936
    python -m cuteafd_b200.bench.microbench moe --tokens 1,16,128,1024,8192 --hidden 7168 --ffn 2048 \
        --experts 256 --top-k 8 --scoring sigmoid

Small kernels (a few microseconds) are timed as a CUDA graph of many launches cycling over more
weight copies than fit in L2, so host launch cost does not pollute the number.  Roofline
denominators come from MEASURED_PEAKS.json at the repository root when present (measured copy
bandwidth and cuBLAS bf16 throughput), else 6650 GB/s and 1590 TFLOP/s.

The MoE mode is the dispatch -> expert -> combine benchmark of the reference's exchange path
(rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2489-2512 plus the expert worker), here
plan + dispatch + grouped fc1/SwiGLU + grouped fc2/combine kernels on one GPU or, under torchrun,
with the experts on the other ranks.
"""
from __future__ import annotations

import argparse
import json
import os

import torch

from ..ops import kernels as K

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def peaks() -> dict:
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "kind": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "kind": "fallback"}


_flush = None


def flush_l2(dev) -> None:
    global _flush
    if _flush is None:
        _flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
    _flush.zero_()


def time_eager(fn, dev, iters: int = 10, warm: int = 3) -> float:
    """Median milliseconds of one call, L2 flushed before each timed call."""
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(iters):
        flush_l2(dev)
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); fn(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2]


def time_graph(fns, reps: int = 5) -> float:
    """Median milliseconds per call for a list of calls captured into one CUDA graph."""
    for f in fns:
        f()
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        for f in fns:
            f()
    g.replay()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record(); g.replay(); b.record()
        torch.cuda.synchronize()
        ts.append(a.elapsed_time(b))
    return sorted(ts)[len(ts) // 2] / len(fns)


def report(name: str, ms: float, flops: float, byts: float, pk: dict) -> dict:
    tf, gb = flops / ms / 1e9, byts / ms / 1e6
    r = {"case": name, "us": round(ms * 1e3, 2), "tflops": round(tf, 1), "gbs": round(gb, 0),
         "frac_compute": round(tf / pk["bf16_tflops"], 3), "frac_hbm": round(gb / pk["hbm_gbs"], 3), "of": pk["kind"]}
    print(json.dumps(r), flush=True)
    return r


def bench_gemm(a, dev, pk):
    T, N, Kd = a.tokens, a.features, a.k
    x = torch.randn(T, Kd, device=dev).bfloat16()
    out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    per = N * Kd * 2 * (2 if a.dual else 1)
    copies = 1 if T > 256 else max(2, min(24, int(200e6 // per) + 1))
    ws = [(torch.randn(N, Kd, device=dev) * 0.02).bfloat16() for _ in range(copies)]
    us = [(torch.randn(N, Kd, device=dev) * 0.02).bfloat16() if a.dual else None for _ in range(copies)]
    if T > 256:
        ms = time_eager(lambda: K.linear(x, ws[0], out=out, w_up=us[0]), dev, iters=a.iters)
    else:
        ms = time_graph([(lambda w=w, u=u: K.linear(x, w, out=out, w_up=u)) for w, u in zip(ws, us)] * 2)
    flops = 2.0 * T * N * Kd * (2 if a.dual else 1)
    report(f"gemm T={T} N={N} K={Kd} dual={a.dual}", ms, flops, per + (T * Kd + T * N) * 2, pk)
    assert K.read_status() == 0


def bench_attn_prefill(a, dev, pk):
    Hq, Hkv, D, n = a.heads, a.kv_heads, 128, a.len
    pages = (n + 63) // 64 + 1
    kc = torch.randn(pages, Hkv, 64, D, device=dev).bfloat16()
    vc = torch.randn_like(kc)
    kc[0] = 0; vc[0] = 0
    table = torch.arange(1, pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
    q = torch.randn(n, Hq, D, device=dev).bfloat16()
    out = torch.empty_like(q)
    sl = torch.tensor([n], dtype=torch.int32, device=dev)
    qs = torch.tensor([0, n], dtype=torch.int32, device=dev)
    w = a.window
    ms = time_eager(lambda: K.attn_prefill(q, kc, vc, table, sl, qs, out, n, window=w), dev, iters=a.iters)
    # visible (query, key) pairs: the causal triangle, or the band of a sliding window
    pairs = n * n / 2 if not w or w >= n else n * w - w * w / 2
    report(f"attn_prefill len={n} Hq={Hq} Hkv={Hkv}" + (f" window={w}" if w else ""), ms, 4.0 * pairs * D * Hq,
           (2 * n * Hq * D + 2 * n * Hkv * D) * 2, pk)
    assert K.read_status() == 0


def bench_attn_decode(a, dev, pk):
    Hq, Hkv, D, S, n = a.heads, a.kv_heads, 128, a.seqs, a.len
    pps = (n + 63) // 64
    pages = S * pps + 1
    kcs = [torch.randn(pages, Hkv, 64, D, device=dev).bfloat16() for _ in range(2 if S >= 16 else 4)]
    table = (torch.arange(S * pps, dtype=torch.int32, device=dev) + 1).view(S, pps).contiguous()
    q = torch.randn(S, Hq, D, device=dev).bfloat16()
    out = torch.empty_like(q)
    sl = torch.full((S,), n, dtype=torch.int32, device=dev)
    qs = torch.arange(S + 1, dtype=torch.int32, device=dev)
    splits = a.splits or K.attn_decode_splits(S, 1, Hkv, pps, a.window)
    scratch = torch.empty(K.attn_decode_scratch_floats(S, 1, Hq, Hkv, splits), dtype=torch.float32, device=dev)
    w = a.window
    seen = min(n, w) if w else n                                       # positions a row reads
    ms = time_graph([(lambda kc=kc: K.attn_decode(q, kc, kc, table, sl, qs, out, scratch, 1, splits, window=w)) for kc in kcs] * 3)
    report(f"attn_decode seqs={S} len={n} splits={splits}" + (f" window={w}" if w else ""), ms, 4.0 * S * seen * D * Hq,
           S * seen * Hkv * D * 2 * 2.0, pk)


def bench_moe(a, dev, pk):
    from ..parallel.moe_exchange import ExchangeGeometry, LocalExchange
    H, I, E, k = a.hidden, a.ffn, a.experts, a.top_k
    sets = []
    n_sets = 1 if E * 3 * H * I * 2 > 2e9 else 2
    for _ in range(n_sets):
        sets.append(tuple((torch.randn(E, r, c, device=dev) * 0.02).bfloat16() for r, c in ((I, H), (I, H), (H, I))))
    kw = dict(scoring=a.scoring, num_groups=a.groups, topk_groups=a.topk_groups)
    for T in [int(t) for t in a.tokens.split(",")]:
        ex = LocalExchange(ExchangeGeometry(H, I, E, k, T, 1), dev)
        x = torch.randn(T, H, device=dev).bfloat16()
        res = torch.randn(T, H, device=dev).bfloat16()
        logits = torch.randn(T, E, device=dev)
        out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        fns = [(lambda s=s: ex.forward(x, logits, kw, s[0], s[1], s[2], out, residual=res)) for s in sets]
        if T <= 256:
            ms = time_graph(fns * 3)
        else:
            ms = time_eager(fns[0], dev, iters=a.iters)
        idx = ex.att.idx[:T]
        active = int(torch.unique(idx).numel())
        byts = active * 3 * H * I * 2 + T * k * H * 2 * 2 + T * k * I * 2 * 2 + T * k * H * 2 * 2
        report(f"moe T={T} H={H} I={I} E={E} k={k} active={active}", ms, 2.0 * T * k * 3 * H * I, byts, pk)
        assert K.read_status() == 0


def bench_mla(a, dev, pk):
    """Absorbed MLA attention: decode (one row per sequence) when --qlen 1, prefill / verify rows otherwise."""
    import math
    heads, S, n, ql = a.heads, a.seqs, a.len, a.qlen
    pps = (n + 63) // 64
    pages = S * pps + 1
    caches = [torch.randn(pages, 64, 576, device=dev).bfloat16() for _ in range(1 if pages * 64 * 576 * 2 > 150e6 else 3)]
    table = (torch.arange(S * pps, dtype=torch.int32, device=dev) + 1).view(S, pps).contiguous()
    T = S * ql
    q = (torch.randn(T, heads, 576, device=dev) * 0.3).bfloat16()
    out = torch.empty(T, heads, 512, dtype=torch.bfloat16, device=dev)
    sl = torch.full((S,), n, dtype=torch.int32, device=dev)
    qs = torch.arange(S + 1, dtype=torch.int32, device=dev) * ql
    i32 = dict(dtype=torch.int32, device=dev)
    sparse = None
    if a.topk:
        base = torch.arange(a.topk, **i32) * max(1, n // a.topk)
        sparse = base[None, :].repeat(T, 1).contiguous()
        bs, bt = K.mla_blocks([ql] * S, 128)
    else:
        bs, bt = K.mla_blocks([ql] * S, heads)
    nb = len(bs)
    tiles = (a.topk or n) // 32
    splits = a.splits or max(1, min(K.num_sms() // max(1, nb * 2), max(1, tiles // 8), 32))
    scratch = torch.empty(K.mla_scratch_floats(nb, splits), dtype=torch.float32, device=dev) if splits > 1 else None
    bsd, btd = torch.tensor(bs, **i32), torch.tensor(bt, **i32)
    scale = 1.0 / math.sqrt(192)
    fns = [(lambda c=c: K.mla_attention(q, c, table, sl, qs, bsd, btd, out, scale, splits, scratch, sparse_idx=sparse)) for c in caches]
    ms = time_graph(fns * 3) if T <= 512 else time_eager(fns[0], dev, iters=a.iters)
    kv = a.topk or n
    avg_kv = kv if (ql == 1 or a.topk) else (n - ql / 2)
    flops = 2.0 * T * heads * avg_kv * (576 + 512)
    byts = (S * n if not a.topk else T * kv) * 576 * 2.0 + T * heads * (576 + 512) * 2.0
    report(f"mla seqs={S} len={n} qlen={ql} heads={heads} topk={a.topk} splits={splits}", ms, flops, byts, pk)
    assert K.read_status() == 0


def bench_mla_prefill_expanded(a, dev, pk):
    """MLA prefill in expanded form (per-head K_nope / V from kv_b, shared rope keys from the latent cache)."""
    import math
    heads, n = a.heads, a.len
    pages = (n + 63) // 64 + 1
    cache = torch.randn(pages, 64, 576, device=dev).bfloat16(); cache[0] = 0
    table = torch.arange(1, pages, dtype=torch.int32, device=dev).view(1, -1).contiguous()
    q = (torch.randn(n, heads * 192, device=dev) * 0.3).bfloat16()
    qr = (torch.randn(n, heads, 576, device=dev) * 0.3).bfloat16()
    rows = ((n + 63) // 64) * 64
    kx = (torch.randn(rows, heads * 128, device=dev) * 0.3).bfloat16(); vx = torch.randn_like(kx)
    out = torch.empty(n, heads, 128, dtype=torch.bfloat16, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    sl, qs, z = torch.tensor([n], **i32), torch.tensor([0, n], **i32), torch.zeros(1, **i32)
    ms = time_eager(lambda: K.attn_prefill_mla(q, qr, kx, vx, z, cache, table, sl, qs, out, n, heads, 1.0 / math.sqrt(192)), dev, iters=a.iters)
    report(f"mla_prefill_expanded len={n} heads={heads}", ms, 2.0 * n * n / 2 * heads * (192 + 128), (n * heads * (192 + 128 + 256)) * 2.0, pk)
    assert K.read_status() == 0


def bench_w4(a, dev, pk):
    """4-bit weight GEMM at decode sizes against the bf16 kernel on the same logical weights."""
    from ..quant import codecs
    T, N, Kd = a.tokens, a.features, a.k
    x = torch.randn(T, Kd, device=dev).bfloat16()
    out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    copies = max(2, min(16, int(300e6 // (N * Kd // 2)) + 1))
    g = torch.Generator().manual_seed(0)
    w = torch.randn(N, Kd, generator=g) * 0.05
    if a.fmt == "mxfp4":
        pq, sq = codecs.mxfp4_quant(w)
        ws = [(pq.to(dev).clone(), sq.to(dev).clone(), None) for _ in range(copies)]
    else:
        pq, sq, gq = codecs.nvfp4_quant(w)
        ws = [(pq.to(dev).clone(), sq.view(torch.uint8).to(dev).clone(), gq.to(dev)) for _ in range(copies)]
    ms = time_graph([(lambda w_=w_: K.linear_w4(x, w_, a.fmt, out=out)) for w_ in ws] * 2)
    per = N * Kd // 2 + N * Kd // (32 if a.fmt == "mxfp4" else 16)
    report(f"gemm_w4 {a.fmt} T={T} N={N} K={Kd}", ms, 2.0 * T * N * Kd, per + (T * Kd + T * N) * 2, pk)
    wb = [(torch.randn(N, Kd, device=dev) * 0.05).bfloat16() for _ in range(max(2, copies // 4))]
    ms_b = time_graph([(lambda w_=w_: K.linear(x, w_, out=out)) for w_ in wb] * 2)
    report(f"gemm bf16 twin T={T} N={N} K={Kd}", ms_b, 2.0 * T * N * Kd, N * Kd * 2 + (T * Kd + T * N) * 2, pk)
    assert K.read_status() == 0


def bench_exl3(a, dev, pk):
    """EXL3 trellis GEMM at decode sizes (Hadamard rotations + in-kernel trellis decode + tcgen05)."""
    from ..quant import codecs
    T, N, Kd, bits = a.tokens, a.features, a.k, a.bits
    x = torch.randn(T, Kd, device=dev).bfloat16()
    copies = max(2, min(16, int(300e6 // (N * Kd * bits // 8)) + 1))
    g = torch.Generator().manual_seed(0)
    ws = []
    for _ in range(copies):
        t, su, sv = codecs.exl3_random(Kd, N, bits, g)
        ws.append((t.to(dev), su.to(dev), sv.to(dev)))
    out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    ms = time_graph([(lambda w=w: K.linear_exl3(x, w[0], w[1], w[2], out=out)) for w in ws] * 2)
    per = N * Kd * bits // 8 + (N + Kd) * 2
    report(f"gemm_exl3 k{bits} T={T} N={N} K={Kd}", ms, 2.0 * T * N * Kd, per + (T * Kd + T * N) * 2, pk)
    assert K.read_status() == 0


def bench_gemm_fp8(a, dev, pk):
    """Block-scaled E4M3 GEMM (128 x 128 weight scales, 1 x 128 activation scales)."""
    from ..quant import codecs
    T, N, Kd = a.tokens, a.features, a.k
    x = torch.randn(T, Kd, device=dev).bfloat16()
    xq = torch.empty(T, Kd, dtype=torch.float8_e4m3fn, device=dev)
    xs = torch.empty(T, Kd // 128, dtype=torch.float32, device=dev)
    K.quant_rows_fp8(x, xq, xs)
    copies = 1 if T > 256 else max(2, min(24, int(200e6 // (N * Kd)) + 1))
    ws = []
    for i in range(copies):
        q, sc = codecs.fp8_quant_block128(torch.randn(N, Kd, generator=torch.Generator().manual_seed(i)) * 0.05)
        ws.append((q.to(dev), sc.to(dev)))
    out = torch.empty(T, N, dtype=torch.bfloat16, device=dev)
    if T > 256:
        ms = time_eager(lambda: K.linear_fp8(xq, xs, ws[0][0], ws[0][1], out=out), dev, iters=a.iters)
    else:
        ms = time_graph([(lambda w=w: K.linear_fp8(xq, xs, w[0], w[1], out=out)) for w in ws] * 2)
    report(f"gemm_fp8 T={T} N={N} K={Kd}", ms, 2.0 * T * N * Kd, N * Kd + T * Kd + T * N * 2, pk)
    assert K.read_status() == 0


def bench_indexer(a, dev, pk):
    """Lightning indexer: scores of every cached position for each query token, then the radix top-k."""
    heads, S, n, topk = a.heads, a.seqs, a.len, a.topk
    pps = (n + 63) // 64
    pages = S * pps + 1
    kc = torch.randn(pages, 64, 128, device=dev).bfloat16()
    table = (torch.arange(S * pps, dtype=torch.int32, device=dev) + 1).view(S, pps).contiguous()
    q = (torch.randn(S, heads, 128, device=dev) * 0.3).bfloat16()
    hw = torch.rand(S, heads, device=dev).bfloat16()
    sl = torch.full((S,), n, dtype=torch.int32, device=dev)
    qs = torch.arange(S + 1, dtype=torch.int32, device=dev)
    bs, bt = K.mla_blocks([1] * S, heads // 2)
    i32 = dict(dtype=torch.int32, device=dev)
    bsd, btd = torch.tensor(bs, **i32), torch.tensor(bt, **i32)
    ld = ((pps * 64 + 127) // 128) * 128
    scores = torch.empty(S, ld, dtype=torch.float32, device=dev)
    sel = torch.empty(S, topk, dtype=torch.int32, device=dev)
    splits = max(1, min(K.num_sms() // max(1, len(bs)), max(1, (pps + 1) // 4), 64))
    ms = time_graph([lambda: K.indexer_scores(q, kc, hw, table, sl, qs, bsd, btd, scores, splits, w_scale=heads ** -0.5)] * 6)
    report(f"indexer_scores seqs={S} len={n} heads={heads} splits={splits}", ms, 2.0 * S * heads * n * 128, S * n * 128 * 2.0, pk)
    ms2 = time_graph([lambda: K.index_topk(scores, topk, sel, seq_lens=sl, q_start=qs)] * 6)
    report(f"index_topk seqs={S} len={n} k={topk}", ms2, 0.0, S * n * 4.0, pk)
    assert K.read_status() == 0


def bench_sampler(a, dev, pk):
    from ..runtime.sampling import SamplingParams
    n, V = a.rows, a.vocab
    logits = torch.randn(n, V, device=dev) * 3
    params = [SamplingParams(temperature=0.8, top_k=a.top_k or None, top_p=a.top_p, seed=i) for i in range(n)]
    rows = K.pack_sample_rows(params, list(range(n))).to(dev)
    tok = torch.empty(n, dtype=torch.int32, device=dev); st = torch.empty(n, dtype=torch.int32, device=dev)
    ms = time_graph([lambda: K.sample_rows(logits, rows, tok, st)] * 8)
    report(f"sample_rows rows={n} V={V} top_k={a.top_k} top_p={a.top_p}", ms, 0.0, n * V * 4.0, pk)


def main() -> None:
    ap = argparse.ArgumentParser()
    sub = ap.add_subparsers(dest="cmd", required=True)
    ex = sub.add_parser("exl3")
    ex.add_argument("--tokens", type=int, default=8); ex.add_argument("--features", type=int, default=7168)
    ex.add_argument("--k", type=int, default=2048); ex.add_argument("--bits", type=int, default=4)
    f8 = sub.add_parser("gemm-fp8")
    f8.add_argument("--tokens", type=int, default=8); f8.add_argument("--features", type=int, default=7168)
    f8.add_argument("--k", type=int, default=2048); f8.add_argument("--iters", type=int, default=10)
    ix = sub.add_parser("indexer")
    ix.add_argument("--seqs", type=int, default=8); ix.add_argument("--len", type=int, default=32768)
    ix.add_argument("--heads", type=int, default=64); ix.add_argument("--topk", type=int, default=2048)
    g = sub.add_parser("gemm")
    g.add_argument("--tokens", type=int, default=8192); g.add_argument("--features", type=int, default=5120)
    g.add_argument("--k", type=int, default=2048); g.add_argument("--dual", action="store_true")
    p = sub.add_parser("attn-prefill")
    p.add_argument("--len", type=int, default=8192); p.add_argument("--heads", type=int, default=32)
    p.add_argument("--kv-heads", type=int, default=4); p.add_argument("--window", type=int, default=0, help="sliding window in tokens (0 = none)")
    d = sub.add_parser("attn-decode")
    d.add_argument("--seqs", type=int, default=32); d.add_argument("--len", type=int, default=8192)
    d.add_argument("--heads", type=int, default=32); d.add_argument("--kv-heads", type=int, default=4)
    d.add_argument("--splits", type=int, default=0); d.add_argument("--window", type=int, default=0, help="sliding window in tokens (0 = none)")
    m = sub.add_parser("moe")
    m.add_argument("--tokens", default="1,16,128,1024,8192"); m.add_argument("--hidden", type=int, default=2048)
    m.add_argument("--ffn", type=int, default=768); m.add_argument("--experts", type=int, default=128)
    m.add_argument("--top-k", type=int, default=8); m.add_argument("--scoring", default="softmax")
    m.add_argument("--groups", type=int, default=1); m.add_argument("--topk-groups", type=int, default=1)
    ml = sub.add_parser("mla")
    ml.add_argument("--seqs", type=int, default=8); ml.add_argument("--len", type=int, default=8192)
    ml.add_argument("--qlen", type=int, default=1); ml.add_argument("--heads", type=int, default=128)
    ml.add_argument("--topk", type=int, default=0); ml.add_argument("--splits", type=int, default=0)
    mp_ = sub.add_parser("mla-prefill")
    mp_.add_argument("--len", type=int, default=8192); mp_.add_argument("--heads", type=int, default=128)
    w4 = sub.add_parser("w4")
    w4.add_argument("--tokens", type=int, default=8); w4.add_argument("--features", type=int, default=7168)
    w4.add_argument("--k", type=int, default=2048); w4.add_argument("--fmt", default="mxfp4")
    sm = sub.add_parser("sampler")
    sm.add_argument("--rows", type=int, default=32); sm.add_argument("--vocab", type=int, default=151936)
    sm.add_argument("--top-k", type=int, default=50); sm.add_argument("--top-p", type=float, default=0.9)
    for s in (g, p, d, m, ml, mp_, w4, sm):
        s.add_argument("--iters", type=int, default=10)
    a = ap.parse_args()
    dev = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(dev)
    pk = peaks()
    {"exl3": bench_exl3, "gemm-fp8": bench_gemm_fp8, "indexer": bench_indexer, "gemm": bench_gemm, "attn-prefill": bench_attn_prefill, "attn-decode": bench_attn_decode, "moe": bench_moe,
     "mla": bench_mla, "mla-prefill": bench_mla_prefill_expanded, "w4": bench_w4, "sampler": bench_sampler}[a.cmd](a, dev, pk)


if __name__ == "__main__":
    main()
