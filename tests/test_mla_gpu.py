"""Absorbed MLA attention kernel (tcgen05, paged latent cache) against fp32 PyTorch math."""
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module")
def K():
    from cuteafd_b200.ops import kernels
    return kernels


def _dev():
    return torch.device("cuda", 0)


def _latent_cache(lens, seed=0):
    """Random paged latent cache; returns (cache [pages,64,576], table, dense list of [len,576])."""
    g = torch.Generator().manual_seed(seed)
    S = len(lens)
    max_pages = max((n + 63) // 64 for n in lens) + 1
    total = 1 + sum((n + 63) // 64 for n in lens)
    cache = torch.zeros(total, 64, 576, dtype=torch.bfloat16)
    table = torch.zeros(S, max_pages, dtype=torch.int32)
    perm = (torch.randperm(total - 1, generator=g) + 1).tolist()
    dense, nxt = [], 0
    for s, n in enumerate(lens):
        c = (torch.randn(n, 576, generator=g) * 0.5).to(torch.bfloat16)
        dense.append(c)
        for pi in range((n + 63) // 64):
            pg = perm[nxt]; nxt += 1
            table[s, pi] = pg
            rows = c[pi * 64:(pi + 1) * 64]
            cache[pg, :rows.shape[0]] = rows
    return cache.to(_dev()), table.to(_dev()), dense


def _ref(q, c, prior, scale):
    """q [n, heads, 576], c [len, 576] fp32 math; token i sees positions <= prior + i."""
    n = q.shape[0]
    s = torch.einsum("nhd,ld->nhl", q.float(), c.float()) * scale
    pos = torch.arange(c.shape[0])[None, None, :]
    lim = (prior + torch.arange(n))[:, None, None]
    s = s.masked_fill(pos > lim, float("-inf"))
    return torch.einsum("nhl,ld->nhd", torch.softmax(s, -1), c[:, :512].float())


@pytest.mark.parametrize("heads,lens,qlens,splits", [
    (16, [100], [1], 1),
    (16, [700, 64, 1, 333], [1, 1, 1, 1], 4),
    (128, [65, 2000], [1, 1], 8),
    (64, [300], [300], 1),
    (16, [517, 130], [517, 66], 1),
    (128, [200], [3], 2),
    (32, [1000, 40], [5, 40], 3),
])
def test_mla_attention(K, heads, lens, qlens, splits):
    cache, table, dense = _latent_cache(lens, seed=heads + len(lens))
    g = torch.Generator().manual_seed(7)
    T = sum(qlens)
    q = (torch.randn(T, heads, 576, generator=g) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(192)
    bs, bt = K.mla_blocks(qlens, heads)
    dev = _dev()
    i32 = dict(dtype=torch.int32, device=dev)
    q_start = torch.tensor([0] + torch.tensor(qlens).cumsum(0).tolist(), **i32)
    out = torch.full((T, heads, 512), 7.0, dtype=torch.bfloat16, device=dev)
    scratch = torch.empty(K.mla_scratch_floats(len(bs), splits), dtype=torch.float32, device=dev) if splits > 1 else None
    for _ in range(2):                      # twice: barriers, TMEM and scratch are reused cleanly
        K.mla_attention(q.to(dev), cache, table, torch.tensor(lens, **i32), q_start, torch.tensor(bs, **i32),
                        torch.tensor(bt, **i32), out, scale, splits, scratch)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    o = 0
    for s, n in enumerate(qlens):
        ref = _ref(q[o:o + n], dense[s], lens[s] - n, scale)
        got = out[o:o + n].float().cpu()
        err = (got - ref).abs().max().item()
        assert err < 0.03 * max(1.0, ref.abs().max().item()), (s, err)
        o += n


def _mla_cfg():
    from cuteafd_b200.config import ModelConfig
    return ModelConfig(name="mla-moe-small", family="deepseek_v3", vocab_size=2048, num_layers=3, hidden=512,
                       attention="mla", num_heads=16, q_lora_rank=256, kv_lora_rank=512, qk_nope_dim=128, qk_rope_dim=64,
                       v_head_dim=128, rope_theta=10000.0, rope_interleaved=True, dense_ffn=1024, first_dense_layers=1,
                       num_experts=16, expert_ffn=256, top_k=4, scoring="sigmoid", num_groups=4, topk_groups=2,
                       num_shared_experts=1, routed_scale=2.5, router_bias=True)


@pytest.mark.parametrize("use_graphs,indexer", [(False, False), (True, False), (False, True), (True, True),
                                                (False, "fp8"), (True, "fp8"), (True, "twins")])
def test_mla_engine_matches_oracle(K, use_graphs, indexer):
    from cuteafd_b200.models.mla_moe import LatentCache, MlaMoeEngine, MlaMoeWeights
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    cfg = _mla_cfg()
    twins, indexer = indexer == "twins", (False if indexer == "twins" else indexer)
    if indexer:                                   # sparse attention: 48 of up to ~200 cached positions per token
        cfg = cfg.replace(family="deepseek_v32", indexer_heads=32, indexer_dim=128, indexer_topk=48)
    if indexer == "fp8":                          # 656-byte FP8 latent records, expanded per step for the sparse kernel
        cfg = cfg.replace(kv_format="fp8_ds_mla", indexer_topk=64)
    dev = _dev()
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    W = MlaMoeWeights.from_params(cfg, params, dev)
    if twins:
        # E4M3 twins of q_b, the o projection and the shared expert for decode-sized steps (prompt chunks stay on bf16)
        from cuteafd_b200.loader.load import attach_fp8_twins
        assert attach_fp8_twins(W) == 2 * cfg.num_layers + 3 * (cfg.num_layers - cfg.first_dense_layers)
        assert set(W.layers[1].fp8) == {"wq_b", "wo", "s_gate", "s_up", "s_down"} and W.layers[1].fp8["wo"][0].dtype == torch.float8_e4m3fn
    eng = MlaMoeEngine(cfg, W, LatentCache(cfg, 64, dev), max_tokens=256, max_seqs=8)
    gen = Generator(eng, PagePool(64), max_pages_per_seq=8, max_seqs=8, prefill_chunk=128, use_graphs=use_graphs)
    ref = RefDecoder(cfg, params)
    # Index scores of near-tied positions flip with bf16 noise, so in eager mode the oracle attends to the
    # positions the engine selected (and the two selections are compared); under graphs only a loose bound holds.
    forced = indexer and not use_graphs
    picked, agree = {}, []
    if forced:
        eng.select_hook = lambda layer, sel: picked.setdefault(layer, []).append(sel.cpu())

        def select_fn(layer, start, Tq, Tk, own):
            sel = picked[layer].pop(0)            # selections arrive in the order the engine ran its forward passes
            assert sel.shape[0] == Tq
            m = torch.zeros(Tq, Tk, dtype=torch.bool)
            for i in range(Tq):
                m[i, sel[i][sel[i] >= 0].long()] = True
            agree.append(((m & own).sum().float() / own.sum().float()).item())      # shared share of the selected positions
            return m
        ref.select_fn = select_fn
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (200, 77)]
    seqs, last, ref_kv, errs = [], [], [], []
    with torch.no_grad():
        for p in prompts:
            s = gen.table.new()
            picked.clear()
            gen.prefill(s, p.tolist())
            kvs = KvState(cfg)
            if forced:                            # the oracle sees the prompt in the same chunks as the engine
                for c0 in range(0, len(p), 128):
                    rl = ref.forward(p[c0:c0 + 128], kvs)[-1]
            else:
                rl = ref.forward(p, kvs)[-1]
            got = eng.logits[0].float().cpu()
            err = (got - rl).abs().max().item() / max(rl.abs().max().item(), 1.0)
            if indexer and not forced:
                errs.append(err)
            else:
                assert err < 0.05, err
            seqs.append(s); ref_kv.append(kvs)
            last.append(int(rl.argmax()))
        for step in range(5):
            picked.clear()
            gen.decode(seqs, last)
            torch.cuda.synchronize()
            assert K.read_status() == 0
            rows = {layer: v[0] for layer, v in picked.items()}
            for i in range(len(seqs)):
                for layer in rows:
                    picked[layer] = [rows[layer][i:i + 1]]
                rl = ref.forward(torch.tensor([last[i]]), ref_kv[i])[-1]
                got = eng.logits[i].float().cpu()
                errs.append((got - rl).abs().max().item() / max(rl.abs().max().item(), 1.0))
                last[i] = int(rl.argmax())
    errs.sort()
    if twins:
        # the oracle keeps the projections in bf16: E4M3 weights and 1x128 activation scales add a few per cent
        assert errs[len(errs) // 2] < 0.08 and errs[-1] < 0.3, errs
    elif indexer and not forced:
        assert errs[len(errs) // 2] < 0.15 and errs[-1] < 0.4, errs
    else:
        # the absorbed form rounds at different points than the oracle's expanded form, so a near-tie in the
        # sigmoid router can pick another expert for a row: most rows must agree tightly, none may be far off
        assert errs[len(errs) // 2] < 0.03 and errs[-3] < 0.05 and errs[-1] < 0.25, errs
    if forced:
        assert sum(agree) / len(agree) > 0.95 and min(agree) > 0.8, agree


@pytest.mark.parametrize("heads,n", [(16, 128), (16, 300), (128, 200)])
def test_mla_prefill_expanded_form(K, heads, n):
    """Expanded-form MLA prefill kernel: per-head 128-dim keys/values plus a 64-dim rope part shared by all heads."""
    g = torch.Generator().manual_seed(heads + n)
    dev = _dev()
    cache, table, dense = _latent_cache([n], seed=5)
    q = (torch.randn(n, heads, 192, generator=g) * 0.5).to(torch.bfloat16)
    qr_buf = torch.zeros(n, heads, 576, dtype=torch.bfloat16)
    qr_buf[:, :, 512:] = q[:, :, 128:]
    rows = ((n + 63) // 64) * 64
    kx = torch.zeros(rows, heads, 128, dtype=torch.bfloat16); vx = torch.zeros(rows, heads, 128, dtype=torch.bfloat16)
    kx[:n] = (torch.randn(n, heads, 128, generator=g) * 0.5).to(torch.bfloat16)
    vx[:n] = (torch.randn(n, heads, 128, generator=g) * 0.5).to(torch.bfloat16)
    scale = 1.0 / math.sqrt(192)
    out = torch.full((n, heads, 128), 7.0, dtype=torch.bfloat16, device=dev)
    i32 = dict(dtype=torch.int32, device=dev)
    for _ in range(2):
        K.attn_prefill_mla(q.reshape(n, heads * 192).to(dev), qr_buf.to(dev), kx.reshape(rows, -1).to(dev), vx.reshape(rows, -1).to(dev),
                           torch.zeros(1, **i32), cache, table, torch.tensor([n], **i32), torch.tensor([0, n], **i32), out, n, heads, scale)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    k_rope = dense[0][:, 512:].float()                                     # shared across heads
    s = (torch.einsum("nhd,lhd->nhl", q[:, :, :128].float(), kx[:n].float()) +
         torch.einsum("nhd,ld->nhl", q[:, :, 128:].float(), k_rope)) * scale
    mask = torch.arange(n)[None, None, :] > torch.arange(n)[:, None, None]
    ref = torch.einsum("nhl,lhd->nhd", torch.softmax(s.masked_fill(mask, float("-inf")), -1), vx[:n].float())
    err = (out.float().cpu() - ref).abs().max().item()
    assert err < 0.03 * max(1.0, ref.abs().max().item()), err
