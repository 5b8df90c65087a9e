"""Lightning indexer (scores + top-k) and sparse MLA attention against fp32 PyTorch math."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cuteafd_b200.ops import kernels
    return kernels


DEV = torch.device("cuda", 0)


def _paged(lens, width, seed):
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    max_pages = max((n + 63) // 64 for n in lens) + 1
    total = 1 + sum((n + 63) // 64 for n in lens)
    cache = torch.zeros(total, 64, width, dtype=torch.bfloat16)
    table = torch.zeros(S, max_pages, dtype=torch.int32)
    perm = (torch.randperm(total - 1, generator=g) + 1).tolist()
    dense, nxt = [], 0
    for s, n in enumerate(lens):
        c = (torch.randn(n, width, generator=g) * 0.5).to(torch.bfloat16)
        dense.append(c)
        for pi in range((n + 63) // 64):
            pg = perm[nxt]; nxt += 1
            table[s, pi] = pg
            rows = c[pi * 64:(pi + 1) * 64]
            cache[pg, :rows.shape[0]] = rows
    return cache.to(DEV), table.to(DEV), dense


@pytest.mark.parametrize("heads,lens,qlens,splits", [(32, [100], [1], 1), (64, [700, 64, 1, 333], [1, 1, 1, 1], 3),
                                                     (64, [300], [300], 1), (32, [517, 130], [517, 66], 1), (128, [1000], [5], 2)])
def test_indexer_scores(K, heads, lens, qlens, splits):
    cache, table, dense = _paged(lens, 128, seed=heads)
    g = torch.Generator().manual_seed(3)
    T = sum(qlens)
    q = (torch.randn(T, heads, 128, generator=g) * 0.5).to(torch.bfloat16)
    w = (torch.randn(T, heads, generator=g) * 0.2).to(torch.bfloat16)
    i32 = dict(dtype=torch.int32, device=DEV)
    bs, bt = K.mla_blocks(qlens, heads // 2)              # 256 / heads tokens per block
    ld = ((max(lens) + 127) // 128) * 128
    scores = torch.full((T, ld), 123.0, dtype=torch.float32, device=DEV)
    q_start = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), **i32)
    for _ in range(2):
        K.indexer_scores(q.to(DEV), cache, w.to(DEV), table, torch.tensor(lens, **i32), q_start, torch.tensor(bs, **i32),
                         torch.tensor(bt, **i32), scores, splits, w_scale=0.5)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    got = scores.cpu()
    o = 0
    for s, n in enumerate(qlens):
        ref = torch.einsum("th,thl->tl", w[o:o + n].float() * 0.5, torch.relu(torch.einsum("thd,ld->thl", q[o:o + n].float(), dense[s].float())))
        for i in range(n):
            lim = lens[s] - n + i + 1
            err = (got[o + i, :lim] - ref[i, :lim]).abs().max().item()
            assert err < 0.02 * max(1.0, ref[i, :lim].abs().max().item()), (s, i, err)
            tile_end = min(ld, ((lim + 127) // 128) * 128)
            assert torch.isneginf(got[o + i, lim:tile_end]).all()
        o += n


def _topk_ref(row, n, k):
    if n <= k:
        return list(range(n)) + [-1] * (k - n)
    x = row[:n].clone()
    x[torch.isnan(x)] = float("-inf")
    order = torch.sort(x, descending=True, stable=True).indices[:k]       # stable: equal scores keep the lower position first
    return sorted(order.tolist())


def test_index_topk(K):
    g = torch.Generator().manual_seed(0)
    T, ld, k = 9, 5000, 64
    scores = torch.randn(T, ld, generator=g)
    scores[1] = torch.round(scores[1] * 2) / 2            # heavy ties
    scores[2, ::3] = float("-inf")
    scores[3, 10] = float("nan")
    scores[4] = 1.0                                       # all equal: the lowest positions win
    limits = [5000, 4097, 3000, 777, 500, 64, 10, 65, 1]
    out = torch.full((T, k), -9, dtype=torch.int32, device=DEV)
    for _ in range(2):
        K.index_topk(scores.to(DEV), k, out, limits=torch.tensor(limits, dtype=torch.int32, device=DEV))
    torch.cuda.synchronize()
    got = out.cpu().tolist()
    for t in range(T):
        assert got[t] == _topk_ref(scores[t], limits[t], k), t


@pytest.mark.parametrize("T,ld", [(6, 40000), (40, 40000), (20, 70000)])
def test_index_topk_over_a_cluster(K, T, ld):
    """Rows long enough for the selection to spread one row over a cluster of CTAs (6 rows: eight CTAs each, keys in
    registers; 40 rows: one CTA each, streamed; 20 rows of 70000: four CTAs each, streamed): slices that end inside the
    row, a row shorter than the request, ties across slice borders, an all-equal row."""
    g = torch.Generator().manual_seed(1)
    k = 2048
    scores = torch.randn(T, ld, generator=g)
    scores[1] = torch.round(scores[1] * 4) / 4
    scores[2] = 0.5
    scores[3, ::2] = float("-inf")
    scores[5] = torch.relu(scores[5]) * 1e-3            # most entries zero, the rest in a narrow range
    limits = [ld, ld - 1, ld - 7000, ld // 2 + 11, 2048, 9000] + [ld - 13 * i for i in range(T - 6)]
    out = torch.full((T, k), -9, dtype=torch.int32, device=DEV)
    for _ in range(2):
        K.index_topk(scores.to(DEV), k, out, limits=torch.tensor(limits, dtype=torch.int32, device=DEV))
    torch.cuda.synchronize()
    got = out.cpu().tolist()
    for t in list(range(6)) + list(range(6, T, 7)):
        assert got[t] == _topk_ref(scores[t], limits[t], k), t


@pytest.mark.parametrize("heads,lens,qlens,topk,splits", [(128, [300], [1], 64, 1), (64, [900, 70], [1, 1], 128, 2),
                                                         (128, [200], [6], 96, 1), (16, [1500], [3], 512, 4)])
def test_sparse_mla(K, heads, lens, qlens, topk, splits):
    cache, table, dense = _paged(lens, 576, seed=heads + 1)
    g = torch.Generator().manual_seed(11)
    T = sum(qlens)
    q = (torch.randn(T, heads, 576, generator=g) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(192)
    idx = torch.full((T, topk), -1, dtype=torch.int32)
    o = 0
    sel = []
    for s, n in enumerate(qlens):
        for i in range(n):
            lim = lens[s] - n + i + 1
            m = min(lim, topk)
            pos = torch.randperm(lim, generator=g)[:m].sort().values
            idx[o + i, :m] = pos.to(torch.int32)
            sel.append((s, pos))
        o += n
    i32 = dict(dtype=torch.int32, device=DEV)
    bs, bt = K.mla_blocks(qlens, 128)                     # one token per block
    q_start = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), **i32)
    out = torch.full((T, heads, 512), 7.0, dtype=torch.bfloat16, device=DEV)
    scratch = torch.empty(K.mla_scratch_floats(len(bs), splits), dtype=torch.float32, device=DEV) if splits > 1 else None
    for _ in range(2):
        K.mla_attention(q.to(DEV), cache, table, torch.tensor(lens, **i32), q_start, torch.tensor(bs, **i32),
                        torch.tensor(bt, **i32), out, scale, splits, scratch, sparse_idx=idx.to(DEV))
    torch.cuda.synchronize()
    assert K.read_status() == 0
    got = out.float().cpu()
    for t, (s, pos) in enumerate(sel):
        c = dense[s][pos.long()].float()
        p = torch.softmax(q[t].float() @ c.T * scale, -1)
        ref = p @ c[:, :512]
        err = (got[t] - ref).abs().max().item()
        assert err < 0.03 * max(1.0, ref.abs().max().item()), (t, err)


def _fp8_record_ref(latent, rope):
    """[n, 512] bf16 latents + [n, 64] bf16 rope -> (record bytes [n, 656], dequantised latents as bf16)."""
    n = latent.shape[0]
    v = latent.float().view(n, 4, 128)
    scale = v.abs().amax(-1, keepdim=True).clamp_min(1e-12) * (1.0 / 448.0)
    q = (v * (1.0 / scale)).to(torch.float8_e4m3fn)
    rec = torch.cat([q.view(n, 512).view(torch.uint8), scale.view(n, 4).contiguous().view(torch.uint8).view(n, 16),
                     rope.contiguous().view(torch.uint8).view(n, 128)], dim=1)
    return rec, (q.float() * scale).view(n, 512).to(torch.bfloat16)


def test_fp8_latent_record_write(K):
    """mla_prep_a with a uint8 cache writes E4M3 latents, fp32 scales and bf16 rope in the 656-byte layout."""
    g = torch.Generator().manual_seed(3)
    T, ql = 37, 256
    a = (torch.randn(T, ql + 576, generator=g) * 0.7).to(torch.bfloat16).to(DEV)
    qw = (1 + 0.1 * torch.randn(ql, generator=g)).to(torch.bfloat16).to(DEV)
    kw = (1 + 0.1 * torch.randn(512, generator=g)).to(torch.bfloat16).to(DEV)
    inv = (1.0 / (10000.0 ** (torch.arange(0, 64, 2, dtype=torch.float32) / 64))).to(DEV)
    pos = torch.arange(T, dtype=torch.int32, device=DEV) + 5
    slots = (torch.randperm(128, generator=g)[:T].to(torch.int32) + 64).to(DEV)
    slots[3] = -1
    qa = torch.empty(T, ql, dtype=torch.bfloat16, device=DEV)
    bf = torch.zeros(4, 64, 576, dtype=torch.bfloat16, device=DEV)
    f8 = torch.zeros(4, 64, K.FP8_RECORD_BYTES, dtype=torch.uint8, device=DEV)
    K.mla_prep_a(a, ql, qw, kw, inv, pos, slots, qa, bf, 1e-6, True)
    K.mla_prep_a(a, ql, qw, kw, inv, pos, slots, qa, f8, 1e-6, True)
    torch.cuda.synchronize()
    flat_bf, flat_f8 = bf.view(-1, 576).cpu(), f8.view(-1, K.FP8_RECORD_BYTES).cpu()
    for t in range(T):
        sl = int(slots[t])
        if sl < 0:
            continue
        want, _ = _fp8_record_ref(flat_bf[sl:sl + 1, :512], flat_bf[sl:sl + 1, 512:])
        assert torch.equal(flat_f8[sl], want[0]), t
    assert int(flat_f8[:64].sum()) == 0                   # page 0 untouched


@pytest.mark.parametrize("heads,lens,qlens,topk,splits", [(128, [300], [1], 64, 1), (64, [900, 70], [1, 1], 128, 2),
                                                         (16, [1500], [3], 512, 4)])
def test_sparse_mla_over_fp8_records(K, heads, lens, qlens, topk, splits):
    cache, table, dense = _paged(lens, 576, seed=heads + 2)
    # the same pages as FP8 records
    flat = cache.view(-1, 576).cpu()
    rec, deq = _fp8_record_ref(flat[:, :512], flat[:, 512:])
    cache8 = rec.view(cache.shape[0], 64, K.FP8_RECORD_BYTES).to(DEV)
    deq_cache = torch.cat([deq, flat[:, 512:]], dim=1).view_as(cache).to(DEV)
    g = torch.Generator().manual_seed(12)
    T = sum(qlens)
    q = (torch.randn(T, heads, 576, generator=g) * 0.5).to(torch.bfloat16).to(DEV)
    scale = 1.0 / math.sqrt(192)
    idx = torch.full((T, topk), -1, dtype=torch.int32)
    o = 0
    for s, n in enumerate(qlens):
        for i in range(n):
            lim = lens[s] - n + i + 1
            m = min(lim, topk)
            idx[o + i, :m] = torch.randperm(lim, generator=g)[:m].sort().values.to(torch.int32)
        o += n
    idx = idx.to(DEV)
    i32 = dict(dtype=torch.int32, device=DEV)
    bs, bt = K.mla_blocks(qlens, 128)
    bs, bt = torch.tensor(bs, **i32), torch.tensor(bt, **i32)
    q_start = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), **i32)
    sl = torch.tensor(lens, **i32)
    scratch = torch.empty(K.mla_scratch_floats(len(bs), splits), dtype=torch.float32, device=DEV) if splits > 1 else None
    want = torch.zeros(T, heads, 512, dtype=torch.bfloat16, device=DEV)
    K.mla_attention(q, deq_cache, table, sl, q_start, bs, bt, want, scale, splits, scratch, sparse_idx=idx)
    gathered = torch.full((len(bs), topk, 576), 3.0, dtype=torch.bfloat16, device=DEV)
    got = torch.zeros_like(want)
    K.mla_fp8_gather(cache8, idx, table, sl, q_start, bs, bt, gathered)
    K.mla_attention(q, None, table, sl, q_start, bs, bt, got, scale, splits, scratch, sparse_idx=idx, gathered=gathered)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    # the gathered rows are exactly the dequantised records, and attention over them is the same computation
    pt = table.cpu()
    for t in range(T):
        seq = int(bs[t])
        for e in (0, int((idx[t] >= 0).sum()) - 1):
            pos = int(idx[t, e])
            row = deq_cache[int(pt[seq, pos // 64]), pos % 64]
            assert torch.equal(gathered[t, e], row), (t, e)
    assert torch.equal(got, want)
