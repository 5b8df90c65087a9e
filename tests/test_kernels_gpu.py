"""sm_100a kernels against plain PyTorch fp32 references of the same ops."""
import math
import os

import pytest
import torch

from cuteafd_b200.ref import ops as R

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cuteafd_b200.ops import kernels
    return kernels


def dev():
    return torch.device("cuda:0")


def bf(*shape, scale=1.0, seed=0):
    g = torch.Generator(device="cpu").manual_seed(seed)
    return (torch.randn(*shape, generator=g) * scale).to(torch.bfloat16).to(dev())


def close(a, b, rtol=2e-2, atol=2e-2):
    a, b = a.float().cpu(), b.float().cpu()
    err = (a - b).abs().max().item()
    ref = b.abs().max().item()
    assert torch.allclose(a, b, rtol=rtol, atol=atol * max(ref, 1e-3)), f"max err {err} (ref max {ref})"


def close_gemm(y, x, w, extra=None):
    """A GEMM result against the fp32 product with a bound scaled by the contraction: every element within bf16
    output rounding of its reference (2^-7 relative: one rounding plus accumulation-order noise) plus a floor of
    2^-9 * sqrt(K) * rms(x) * rms(w) for elements near zero.  About a tenth of what the generic check allows; one
    dropped or doubled K block (64 columns: an error of about 8 * rms(x) * rms(w)) is far outside it."""
    xf, wf = x.float().cpu(), w.float().cpu()
    ref = xf @ wf.T
    if extra is not None:
        ref = ref + extra.float().cpu()
    floor = 2.0 ** -9 * math.sqrt(xf.shape[1]) * xf.pow(2).mean().sqrt().item() * wf.pow(2).mean().sqrt().item()
    err = (y.float().cpu() - ref).abs()
    bound = 2.0 ** -7 * ref.abs() + floor
    worst = (err / bound).max().item()
    assert worst <= 1.0, f"worst element at {worst:.2f} x its bound (max err {err.max().item()}, K={xf.shape[1]})"


def check_status(K):
    torch.cuda.synchronize()
    assert K.read_status() == 0


@pytest.mark.parametrize("T,N,Kd,swap", [(128, 256, 128, False), (300, 512, 256, False), (8, 256, 512, True),
                                         (33, 384, 2048, True), (1, 128, 64, True), (200, 256, 192, True),
                                         (1000, 1280, 2048, False)])
def test_linear(K, T, N, Kd, swap):
    x, w = bf(T, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    y = K.linear(x, w, swap=swap)
    check_status(K)
    close_gemm(y, x, w)


@pytest.mark.parametrize("T,swap", [(256, False), (5, True), (70, True)])
def test_linear_swiglu_residual_f32(K, T, swap):
    N, Kd = 256, 512
    x, wg, wu = bf(T, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2), bf(N, Kd, scale=0.05, seed=3)
    y = K.linear(x, wg, w_up=wu, swap=swap)
    ref = torch.nn.functional.silu(x.float() @ wg.float().T) * (x.float() @ wu.float().T)
    close(y, ref)
    res = bf(T, N, seed=4)
    y2 = K.linear(x, wg, residual=res, swap=swap)
    close_gemm(y2, x, wg, extra=res)
    y3 = K.linear(x, wg, out_f32=True, swap=swap)
    assert y3.dtype == torch.float32
    close(y3, x.float() @ wg.float().T, rtol=1e-3, atol=1e-3)
    check_status(K)


def test_linear_ragged_features(K):
    T, N, Kd = 40, 200, 128     # N not a multiple of the feature tile
    x, w = bf(T, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    for swap in (True, False):
        close_gemm(K.linear(x, w, swap=swap), x, w)
    check_status(K)


def test_rmsnorm_embed_argmax(K):
    T, H = 37, 2048
    x, w, r = bf(T, H, seed=1), bf(H, seed=2), bf(T, H, seed=3)
    close(K.rmsnorm(x, w, 1e-6), R.rmsnorm(x, w, 1e-6), 1e-2, 1e-2)
    r2 = r.clone()
    y = K.add_rmsnorm(x, r2, w, 1e-6)
    ry, rr = R.add_rmsnorm(x, r, w, 1e-6)
    assert torch.equal(r2, rr)
    close(y, ry, 1e-2, 1e-2)
    table = bf(500, H, seed=5)
    tok = torch.randint(0, 500, (T,), dtype=torch.int32, device=dev())
    assert torch.equal(K.embed(tok, table), table[tok.long()])
    logits = torch.randn(T, 151936, device=dev())
    logits[3, 77] = logits[3, 90000] = 1e9          # tie -> lowest id
    assert torch.equal(K.argmax(logits).long(), torch.argmax(logits, -1)) or K.argmax(logits)[3].item() == 77
    assert K.argmax(logits)[3].item() == 77


@pytest.mark.parametrize("interleaved,norm,rot,bias", [(False, True, 128, False), (True, False, 128, False),
                                                       (False, False, 64, True), (True, True, 64, True), (False, True, 128, True)])
def test_qk_rope_kv(K, interleaved, norm, rot, bias):
    """``rot`` 64: partial rotary (the second half of every head passes through); ``bias``: q / k / v projection bias
    added to the projection's rows (and rounded) before the norm and the rotation."""
    T, Hq, Hkv, D, pages = 70, 8, 2, 128, 6
    qkv = bf(T, (Hq + 2 * Hkv) * D, seed=1)
    qn, kn = (bf(D, seed=2).abs() + 0.5, bf(D, seed=3).abs() + 0.5) if norm else (None, None)
    theta = 1.0e6
    inv = (1.0 / (theta ** (torch.arange(0, rot, 2, dtype=torch.float32) / rot))).to(dev())
    bq = bf((Hq + 2 * Hkv) * D, seed=9) if bias else None
    pos = torch.arange(100, 100 + T, dtype=torch.int32, device=dev())
    perm = torch.randperm(pages * 64)[:T].to(torch.int32).to(dev())
    kc = torch.zeros(pages, Hkv, 64, D, dtype=torch.bfloat16, device=dev())       # [page, kv head, token, D]
    vc = torch.zeros_like(kc)
    q_out = torch.empty(T, Hq, D, dtype=torch.bfloat16, device=dev())
    K.qk_rope_kv(qkv, qn, kn, inv, pos, perm, q_out, kc, vc, Hq, Hkv, D, 1e-6, interleaved, bias=bq)
    rows = (qkv.float() + bq.float()).to(torch.bfloat16) if bias else qkv
    q, k, v = rows.view(T, Hq + 2 * Hkv, D).split([Hq, Hkv, Hkv], dim=1)
    if norm:
        q, k = R.rmsnorm(q, qn, 1e-6), R.rmsnorm(k, kn, 1e-6)
    rq = R.apply_rope(q, pos.long(), theta, interleaved, inv)
    rk = R.apply_rope(k, pos.long(), theta, interleaved, inv)
    if rot < D:                                     # the dims past the rotated ones come out bit for bit
        assert torch.equal(q_out[..., rot:], q[..., rot:])
    close(q_out, rq, 1e-2, 1e-2)
    by_slot = lambda c: c.permute(0, 2, 1, 3).reshape(-1, Hkv, D)               # noqa: E731  slot = page * 64 + token
    close(by_slot(kc)[perm.long()], rk, 1e-2, 1e-2)
    assert torch.equal(by_slot(vc)[perm.long()], v)


@pytest.mark.parametrize("E,k,scoring,groups,keep", [(128, 8, "softmax", 1, 1), (256, 8, "sigmoid", 8, 4),
                                                     (8, 2, "softmax", 1, 1), (64, 6, "sigmoid", 1, 1)])
def test_route_topk(K, E, k, scoring, groups, keep):
    T = 200
    logits = torch.randn(T, E, device=dev())
    bias = torch.randn(E, device=dev()) * 0.1 if scoring == "sigmoid" else None
    idx, w = K.route_topk(logits, k, scoring, bias, groups, keep, True, 2.5)
    ridx, rw = R.route_topk(logits, k, scoring, bias, groups, keep, True, 2.5)
    assert torch.equal(idx.cpu(), ridx.cpu())
    assert torch.allclose(w.cpu(), rw.cpu(), rtol=1e-4, atol=1e-6)


@pytest.mark.parametrize("T,tile", [(5, 16), (64, 16), (300, 64), (1500, 128)])
def test_moe_local_exchange(K, T, tile):
    from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
    H, I, E, k = 512, 256, 16, 4
    geo = ExchangeGeometry(H, I, E, k, max_tokens=T, n_expert_ranks=1)
    ex = LocalExchange(geo, dev())
    x, res = bf(T, H, seed=1), bf(T, H, seed=2)
    wg, wu, wd = bf(E, I, H, scale=0.05, seed=3), bf(E, I, H, scale=0.05, seed=4), bf(E, H, I, scale=0.05, seed=5)
    logits = torch.randn(T, E, device=dev())
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev())
    ex.forward(x, logits, dict(scoring="softmax"), wg, wu, wd, out, residual=res, tile_rows=tile)
    check_status(K)
    idx, w = R.route_topk(logits, k, "softmax")
    parts = R.moe_forward(x, idx, w, wg, wu, wd)
    ref = R.combine_slots(parts, None, res, torch.bfloat16)
    close(out, ref)
    assert int(ex.att.expert_count.sum().item()) == T * k


@pytest.mark.parametrize("T,E,k", [(2500, 16, 4), (3000, 128, 8)])
def test_moe_wide_plan_matches_single_block(K, T, E, k):
    """Prefill-sized steps plan in three launches (count, scan, scatter); the result is the single-block plan's."""
    from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
    assert T * k >= K.WIDE_PLAN_ENTRIES
    H, I = 256, 128
    logits = torch.randn(T, E, device=dev())
    logits[:, 1] -= 50.0                                   # an expert that nobody picks
    outs = []
    for wide in (True, False):
        old = K.WIDE_PLAN_ENTRIES
        K.WIDE_PLAN_ENTRIES = old if wide else 1 << 30
        try:
            ex = LocalExchange(ExchangeGeometry(H, I, E, k, max_tokens=T, n_expert_ranks=1), dev())
            x = bf(T, H, seed=1)
            wg, wu, wd = bf(E, I, H, scale=0.05, seed=3), bf(E, I, H, scale=0.05, seed=4), bf(E, H, I, scale=0.05, seed=5)
            out = torch.empty(T, H, dtype=torch.bfloat16, device=dev())
            ex.forward(x, logits, dict(scoring="softmax"), wg, wu, wd, out, tile_rows=128)
            check_status(K)
            outs.append((ex.att.dest_row[:T * k].clone(), ex.exp.meta.clone(), out.clone(), ex.att.expert_count.clone()))
        finally:
            K.WIDE_PLAN_ENTRIES = old
    for a, b in zip(outs[0], outs[1]):
        assert torch.equal(a, b)
    idx, w = R.route_topk(logits, k, "softmax")
    ref = R.combine_slots(R.moe_forward(x, idx, w, wg, wu, wd), None, None, torch.bfloat16)
    close(outs[0][2], ref)


def _paged_kv(S, lens, Hkv, D, seed=0):
    """Random K/V per sequence scattered over shuffled pages; returns caches, table, dense copies."""
    pages_per = [(n + 63) // 64 for n in lens]
    total = sum(pages_per) + 1
    order = (torch.randperm(total - 1) + 1).tolist()
    kc = torch.zeros(total, Hkv, 64, D, dtype=torch.bfloat16, device=dev())       # [page, kv head, token, D]
    vc = torch.zeros_like(kc)
    table = torch.zeros(S, max(pages_per), dtype=torch.int32)
    dense = []
    for s in range(S):
        k, v = bf(lens[s], Hkv, D, seed=seed + 2 * s), bf(lens[s], Hkv, D, seed=seed + 2 * s + 1)
        dense.append((k, v))
        for j in range(pages_per[s]):
            pg = order.pop()
            table[s, j] = pg
            n = min(64, lens[s] - 64 * j)
            kc[pg, :, :n], vc[pg, :, :n] = k[64 * j:64 * j + n].transpose(0, 1), v[64 * j:64 * j + n].transpose(0, 1)
    return kc, vc, table.to(dev()), dense


@pytest.mark.parametrize("lens,qlens,splits", [([100], [1], 1), ([700, 64, 1, 333], [1, 1, 1, 1], 4),
                                               ([900, 130], [2, 4], 3), ([8192], [1], 16)])
def test_attn_decode(K, lens, qlens, splits):
    Hq, Hkv, D, S = 32, 4, 128, len(lens)
    kc, vc, table, dense = _paged_kv(S, lens, Hkv, D)
    q = bf(sum(qlens), Hq, D, seed=99)
    q_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev())
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev())
    out = torch.zeros_like(q)
    scratch = torch.empty(K.attn_decode_scratch_floats(S, max(qlens), Hq, Hkv, splits), dtype=torch.float32, device=dev())
    K.attn_decode(q, kc, vc, table, seq_lens, q_start, out, scratch, max(qlens), splits)
    o = 0
    for s in range(S):
        k, v = dense[s]
        ref = R.causal_attention(q[o:o + qlens[s]], k, v, lens[s] - qlens[s])
        close(out[o:o + qlens[s]], ref)
        o += qlens[s]


@pytest.mark.parametrize("lens,qlens", [([128], [128]), ([300], [300]), ([1000], [200]), ([517, 130], [517, 66]),
                                        ([2048], [2048])])
def test_attn_prefill(K, lens, qlens):
    Hq, Hkv, D, S = 8, 2, 128, len(lens)
    kc, vc, table, dense = _paged_kv(S, lens, Hkv, D)
    q = bf(sum(qlens), Hq, D, seed=99)
    q_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev())
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev())
    out = torch.zeros_like(q)
    K.attn_prefill(q, kc, vc, table, seq_lens, q_start, out, max(qlens))
    check_status(K)
    o = 0
    for s in range(S):
        k, v = dense[s]
        ref = R.causal_attention(q[o:o + qlens[s]], k, v, lens[s] - qlens[s])
        close(out[o:o + qlens[s]], ref)
        o += qlens[s]


@pytest.mark.parametrize("lens,qlens,splits,window", [([700, 64, 1, 333], [1, 1, 1, 1], 4, 128), ([900, 130], [2, 4], 3, 100),
                                                      ([8192], [1], 16, 4096), ([500], [1], 2, 1), ([300], [3], 1, 1000)])
def test_attn_decode_sliding_window(K, lens, qlens, splits, window):
    """A query at position t sees keys (t - window, t] only; pages before the window are skipped, whatever the split."""
    Hq, Hkv, D, S = 32, 4, 128, len(lens)
    kc, vc, table, dense = _paged_kv(S, lens, Hkv, D)
    q = bf(sum(qlens), Hq, D, seed=99)
    q_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev())
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev())
    out = torch.zeros_like(q)
    scratch = torch.empty(K.attn_decode_scratch_floats(S, max(qlens), Hq, Hkv, splits), dtype=torch.float32, device=dev())
    K.attn_decode(q, kc, vc, table, seq_lens, q_start, out, scratch, max(qlens), splits, window=window)
    o = 0
    for s in range(S):
        k, v = dense[s]
        ref = R.causal_attention(q[o:o + qlens[s]], k, v, lens[s] - qlens[s], window=window)
        close(out[o:o + qlens[s]], ref)
        o += qlens[s]


@pytest.mark.parametrize("lens,qlens,window", [([300], [300], 64), ([1000], [200], 300), ([517, 130], [517, 66], 128),
                                               ([2048], [2048], 1000), ([640], [640], 1), ([400], [400], 5000)])
def test_attn_prefill_sliding_window(K, lens, qlens, window):
    """kv tiles wholly before the first row's window are not loaded; the tiles that straddle a window edge are masked
    from below as well as along the diagonal."""
    Hq, Hkv, D, S = 8, 2, 128, len(lens)
    kc, vc, table, dense = _paged_kv(S, lens, Hkv, D)
    q = bf(sum(qlens), Hq, D, seed=99)
    q_start = torch.tensor([0] + list(torch.tensor(qlens).cumsum(0)), dtype=torch.int32, device=dev())
    seq_lens = torch.tensor(lens, dtype=torch.int32, device=dev())
    out = torch.zeros_like(q)
    K.attn_prefill(q, kc, vc, table, seq_lens, q_start, out, max(qlens), window=window)
    check_status(K)
    o = 0
    for s in range(S):
        k, v = dense[s]
        ref = R.causal_attention(q[o:o + qlens[s]], k, v, lens[s] - qlens[s], window=window)
        close(out[o:o + qlens[s]], ref)
        o += qlens[s]


# ---- FP8 block-scaled -----------------------------------------------------------------------------------
def _fp8_ref(x, w, w_up=None):
    from cuteafd_b200.quant import codecs
    xq, xs = codecs.fp8_quant_rows(x.float())
    wq, ws = codecs.fp8_quant_block128(w.float())
    xd, wd = codecs.fp8_dequant_rows(xq, xs), codecs.fp8_dequant_block128(wq, ws)
    y = xd @ wd.T
    if w_up is not None:
        uq, us = codecs.fp8_quant_block128(w_up.float())
        y = torch.nn.functional.silu(y) * (xd @ codecs.fp8_dequant_block128(uq, us).T)
        return y, (xq, xs, wq, ws, uq, us)
    return y, (xq, xs, wq, ws, None, None)


def test_quant_rows_fp8_matches_codec(K):
    from cuteafd_b200.quant import codecs
    x = bf(37, 512, seed=3)
    q, s = K.quant_rows_fp8(x)
    rq, rs = codecs.fp8_quant_rows(x.float())
    assert torch.allclose(s, rs, rtol=1e-6)
    assert (codecs.fp8_dequant_rows(q, s) - codecs.fp8_dequant_rows(rq, rs)).abs().max() <= 0.07 * x.float().abs().max()


@pytest.mark.parametrize("T,N,Kd,swap,dual", [(8, 256, 512, True, False), (33, 384, 1024, True, True), (200, 256, 256, False, False),
                                             (300, 512, 768, False, True), (1, 128, 2048, True, False), (64, 2048, 7168, True, False)])
def test_linear_fp8(K, T, N, Kd, swap, dual):
    x, w = bf(T, Kd, seed=1), bf(N, Kd, scale=0.05, seed=2)
    wu = bf(N, Kd, scale=0.05, seed=3) if dual else None
    ref, (xq, xs, wq, ws, uq, us) = _fp8_ref(x, w, wu)
    y = K.linear_fp8(xq.contiguous(), xs.contiguous(), wq.contiguous(), ws.contiguous(), w_up=uq, ws_up=us, swap=swap)
    check_status(K)
    close(y, ref)


@pytest.mark.parametrize("T,tile", [(6, 16), (300, 64), (1500, 128)])
def test_moe_fp8_grouped(K, T, tile):
    """Routed experts in FP8: plan/dispatch in bf16, rows quantised on the expert side, fp8 fc1/fc2."""
    from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
    from cuteafd_b200.quant import codecs
    H, I, E, k = 512, 256, 16, 4
    ex = LocalExchange(ExchangeGeometry(H, I, E, k, max_tokens=T, n_expert_ranks=1), dev())
    x, res = bf(T, H, seed=1), bf(T, H, seed=2)
    wg, wu, wd = bf(E, I, H, scale=0.05, seed=3), bf(E, I, H, scale=0.05, seed=4), bf(E, H, I, scale=0.05, seed=5)
    q = {n: [codecs.fp8_quant_block128(w[e].float()) for e in range(E)] for n, w in (("g", wg), ("u", wu), ("d", wd))}
    st = lambda n, i: torch.stack([p[i] for p in q[n]]).contiguous()
    logits = torch.randn(T, E, device=dev())
    out = torch.empty(T, H, dtype=torch.bfloat16, device=dev())
    ex.forward_fp8(x, logits, dict(scoring="softmax"), (st("g", 0), st("g", 1)), (st("u", 0), st("u", 1)), (st("d", 0), st("d", 1)),
                   out, residual=res, tile_rows=tile)
    check_status(K)
    idx, w = R.route_topk(logits, k, "softmax")
    deq = lambda n: torch.stack([codecs.fp8_dequant_block128(*p) for p in q[n]])
    xq, xs = codecs.fp8_quant_rows(x.float())
    xd = codecs.fp8_dequant_rows(xq, xs).to(torch.bfloat16)
    parts = torch.zeros(T, k, H, device=dev())
    for e in range(E):
        rows, slots = (idx == e).nonzero(as_tuple=True)
        if rows.numel():
            h = (torch.nn.functional.silu(xd[rows].float() @ deq("g")[e].T) * (xd[rows].float() @ deq("u")[e].T)).to(torch.bfloat16)
            hq, hs = codecs.fp8_quant_rows(h.float())
            y = codecs.fp8_dequant_rows(hq, hs) @ deq("d")[e].T
            parts[rows, slots] = y.to(torch.bfloat16).float() * w[rows, slots][:, None]
    close(out, R.combine_slots(parts, None, res, torch.bfloat16), 3e-2, 3e-2)


@pytest.mark.parametrize("T,H", [(5, 512), (40, 2048), (300, 7168), (700, 384)])
def test_dispatch_quantises_on_the_wire(K, T, H):
    """Rows dispatched as E4M3 + per-128 scales equal the rows dispatched in bf16 and quantised on arrival, bit for bit
    (single-block plan+dispatch up to 512 entries, the separate dispatch kernel above that)."""
    from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
    E, k, tile = 16, 4, 16
    ex = LocalExchange(ExchangeGeometry(H, 256, E, k, max_tokens=T, n_expert_ranks=1), dev())
    x = bf(T, H, seed=T)
    x[0, :128] = 0                                               # an all-zero block: scale 1, bytes 0
    logits = torch.randn(T, E, device=dev())
    ex.att.dispatch(x, logits, dict(scoring="softmax"), tile, 0, ex.epoch)
    torch.cuda.synchronize()
    rows = int(ex.exp.tile_row0[: int(ex.exp.num_tiles)].max()) + tile
    dst = ex.att.dest_row[: T * k].long()
    wq, ws = K.quant_rows_fp8(ex.exp.slab[:rows].clone())
    ex.exp.slab.zero_()
    ex.att.dispatch(x, None, dict(scoring="softmax"), tile, 0, ex.epoch, wire_fp8=True)
    torch.cuda.synchronize()
    check_status(K)
    assert torch.equal(ex.att.dest_row[: T * k].long(), dst)
    assert torch.equal(ex.exp.wire_q[dst].view(torch.uint8), wq[dst].view(torch.uint8))
    assert torch.equal(ex.exp.wire_s[dst], ws[dst])


# ---- fused decode-step kernels -------------------------------------------------------------------------------
@pytest.mark.parametrize("E,k,scoring,groups,keep,H", [(128, 8, "softmax", 1, 1, 2048), (256, 8, "sigmoid", 8, 4, 1024)])
def test_norm_route_matches_separate_kernels(K, E, k, scoring, groups, keep, H):
    T = 9
    h, lw, rw = bf(T, H, seed=1), bf(H, seed=2) * 0.1 + 1.0, bf(E, H, scale=0.05, seed=3)
    bias = (torch.randn(E, generator=torch.Generator().manual_seed(4)) * 0.01).to(dev()) if scoring == "sigmoid" else None
    kw = dict(scoring=scoring, num_groups=groups, topk_groups=keep, normalize=True, routed_scale=1.5)
    x_ref = K.rmsnorm(h, lw, 1e-6)
    logits_ref = K.linear(x_ref, rw, out_f32=True)
    idx_ref, w_ref = K.route_topk(logits_ref, k, bias=bias, **kw)
    x = torch.empty_like(h)
    idx = torch.empty(T, k, dtype=torch.int32, device=dev()); w = torch.empty(T, k, dtype=torch.float32, device=dev())
    logits = torch.empty(T, E, dtype=torch.float32, device=dev())
    K.norm_route(h, lw, 1e-6, rw, x, idx, w, k, bias=bias, logits_out=logits, **kw)
    check_status(K)
    assert torch.equal(x, x_ref)
    assert (logits - logits_ref).abs().max().item() < 2e-3 * max(1.0, logits_ref.abs().max().item())
    # same selection wherever the two score computations are not within rounding of a tie
    same = (idx.sort(1).values == idx_ref.sort(1).values).all(1).float().mean().item()
    assert same >= 0.8
    rows = (idx == idx_ref).all(1)
    assert torch.allclose(w[rows], w_ref[rows], rtol=2e-3, atol=1e-5)


def test_combine_with_fused_norm(K):
    T, k, H = 7, 4, 2048
    buf, res, nw = bf(T * k, H, seed=1), bf(T, H, seed=2), bf(H, seed=3) * 0.1 + 1.0
    w = torch.rand(T, k, generator=torch.Generator().manual_seed(5)).to(dev())
    out_ref = torch.empty(T, H, dtype=torch.bfloat16, device=dev())
    K.moe_combine(buf, w, out_ref, residual=res)
    x_ref = K.rmsnorm(out_ref, nw, 1e-6)
    out, x = torch.empty_like(out_ref), torch.empty_like(out_ref)
    K.moe_combine(buf, w, out, residual=res, norm_w=nw, eps=1e-6, x_out=x)
    check_status(K)
    assert torch.equal(out, out_ref)
    assert (x.float() - x_ref.float()).abs().max().item() <= 0.02 * x_ref.float().abs().max().item()


def test_bounded_wait_reports_timeout_and_context_survives(K):
    """A flag that nothing ever sets: the wait gives up after its (shortened) limit, records the peer-flag code in
    the status word and returns; later kernels run normally on the same context."""
    from cuteafd_b200.parallel.health import HealthLatch
    K.set_wait_limit_ns(50_000_000)
    try:
        flag = torch.zeros(1, dtype=torch.int32, device=dev())
        epoch = torch.ones(1, dtype=torch.int32, device=dev())
        K.wait_flag(flag.data_ptr(), epoch)
        torch.cuda.synchronize()
        status = K.read_status()
        assert status == 5
        latch = HealthLatch()
        latch.check_device(status, "test wait")
        assert not latch.ok and "peer flag" in latch.reason
        x, w = bf(4, 256, seed=1), bf(256, seed=2)
        y = K.rmsnorm(x, w, 1e-6)
        torch.cuda.synchronize()
        assert torch.isfinite(y.float()).all() and K.read_status() == 0
    finally:
        K.set_wait_limit_ns(2_000_000_000)


def test_fp8_dequant_block128(K):
    from cuteafd_b200.quant import codecs
    w = torch.randn(3, 256, 384, generator=torch.Generator().manual_seed(0)) * 0.05
    qs = [codecs.fp8_quant_block128(w[e]) for e in range(3)]
    q = torch.stack([a for a, _ in qs]).to(dev()); s = torch.stack([b for _, b in qs]).to(dev())
    out = K.fp8_dequant_block128(q, s)
    ref = torch.stack([codecs.fp8_dequant_block128(a, b) for a, b in qs])
    assert (out.float().cpu() - ref.float()).abs().max().item() <= 0.01 * ref.abs().max().item()


# ---- bounds-check build ------------------------------------------------------------------------------------------
_BOUNDS_CHILD = r'''
import json, os, sys
import torch
from cuteafd_b200._native import lib as N
from cuteafd_b200.ops import kernels as K
from cuteafd_b200.parallel.moe_exchange import ExchangeGeometry, LocalExchange
assert N.bounds_check_enabled(), "this process must have loaded the checked library"
dev = torch.device("cuda:0")
T, H, E, k = 40, 512, 16, 4
out = {}
for T in (40, 300):
    ex = LocalExchange(ExchangeGeometry(H, 256, E, k, max_tokens=T, n_expert_ranks=1), dev)
    x = torch.randn(T, H, device=dev).to(torch.bfloat16)
    logits = torch.randn(T, E, device=dev)
    ex.att.dispatch(x, logits, dict(scoring="softmax"), 16, 0, ex.epoch)
    torch.cuda.synchronize()
    clean = N.take_bad_indices()
    good = ex.exp.slab.clone()
    # the same plan against a layout that claims a slab shorter than the plan needs: the checked build refuses the
    # rows past the end (and says which), stores the others, and nothing outside the slab is touched
    rows = int(ex.att.dest_row[: T * k].max()) + 1
    ex.att.layout.max_rows = rows - 3
    ex.exp.slab.zero_()
    # (the dispatch kernel takes the plan as given; the planner itself never hands out a row past ``max_rows``)
    K.moe_dispatch(x, ex.att.idx[:T], ex.att.dest_row, ex.att.layout, ex.epoch, ex.att.done[0:1])
    torch.cuda.synchronize()
    bad = N.take_bad_indices()
    kept = bool(torch.equal(ex.exp.slab[: rows - 3], good[: rows - 3]))
    skipped = bool((ex.exp.slab[rows - 3: rows] == 0).all())
    out[str(T)] = {"clean": clean, "bad": bad, "kept": kept, "skipped": skipped, "rows": rows}
K.read_status()
print("RESULT " + json.dumps(out))
'''


def test_bounds_check_build_catches_a_row_past_the_slab(K):
    """The checked library (CAFD_BOUNDS_CHECK=1, its own process): a dispatch whose plan points past the end of the slab
    records the site and the index and skips those stores; a correct dispatch records nothing."""
    import json
    import subprocess
    import sys
    from cuteafd_b200._native import build
    if not os.path.exists(build.CHECK_LIB):
        pytest.fail("libcuteafd_b200_chk.so is not built (python -m cuteafd_b200._native.build)")
    env = dict(os.environ, CAFD_BOUNDS_CHECK="1")
    r = subprocess.run([sys.executable, "-c", _BOUNDS_CHILD], env=env, capture_output=True, text=True, timeout=300,
                       cwd=os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    assert r.returncode == 0, r.stdout + r.stderr
    out = json.loads(next(ln for ln in r.stdout.splitlines() if ln.startswith("RESULT "))[7:])
    for T, rec in out.items():
        assert rec["clean"] == [] and rec["kept"] and rec["skipped"], (T, rec)
        (site, idx), = rec["bad"]
        assert "slab row" in site and rec["rows"] - 3 <= idx < rec["rows"], (T, rec)


def test_tcp_expert_worker_computes_on_the_gpu(K):
    """The off-box expert worker's CUDA compute (route sort on the host, tcgen05 grouped GEMMs, scatter back to route
    order) against its plain-tensor twin, called directly and through the wire server."""
    import numpy as np
    from cuteafd_b200.parallel import wire
    H, I, n_exp, lo = 512, 256, 6, 10
    g = torch.Generator().manual_seed(4)
    stacks = tuple((torch.randn(n_exp, a, b, generator=g) * 0.05).to(torch.bfloat16) for a, b in ((I, H), (I, H), (H, I)))
    on_gpu = tuple(t.to(dev()).contiguous() for t in stacks)
    cpu_fn = wire.reference_compute(lambda layer: stacks, lo)
    gpu_fn = wire.cuda_compute(lambda layer: on_gpu, lo, "cuda:0", I)
    rng = np.random.default_rng(0)
    for rows, routes in ((5, 9), (40, 150), (300, 1200), (3, 1)):
        x = (torch.randn(rows, H, generator=g)).to(torch.bfloat16)
        row = rng.integers(0, rows, routes).astype(np.int64)
        expert = (lo + rng.integers(0, n_exp - 1, routes)).astype(np.int64)            # the last expert gets no rows
        weight = rng.random(routes).astype(np.float32)
        want = cpu_fn(0, x, row, expert, weight)
        got = gpu_fn(0, x, row, expert, weight)
        check_status(K)
        assert got.shape == want.shape and got.dtype == torch.float32
        close(got, want, 2e-2, 1e-2)
    plan = wire.plan_hash({"m": 1})
    srv = wire.ExpertServer(gpu_fn, plan).start()
    try:
        remote = wire.RemoteExperts([("127.0.0.1", srv.port, lo, lo + n_exp)], plan)
        x = torch.randn(16, H, generator=g).to(torch.bfloat16)
        idx = torch.randint(lo, lo + n_exp, (16, 2), generator=g)
        w = torch.rand(16, 2, generator=g)
        got = remote(0, x, idx, w).sum(1)
        want = sum(cpu_fn(0, x, np.arange(16), idx[:, s].numpy(), w[:, s].numpy()) for s in range(2))
        close(got, want, 2e-2, 1e-2)
        assert srv.served > 0
        remote.close()
    finally:
        srv.stop()
