"""End to end: the CUDA engine against the CPU oracle on a small GQA MoE decoder."""
import pytest
import torch

from cuteafd_b200.config import ModelConfig

pytestmark = pytest.mark.gpu


def small_cfg() -> ModelConfig:
    return ModelConfig(name="gqa-moe-small", family="qwen3_moe", vocab_size=2048, num_layers=3, hidden=512,
                       attention="gqa", num_heads=8, num_kv_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                       rope_interleaved=False, dense_ffn=1024, first_dense_layers=1, num_experts=16, expert_ffn=256,
                       top_k=4, scoring="softmax", num_shared_experts=1)


def build(cfg, use_graphs):
    from cuteafd_b200.models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    dev = torch.device("cuda:0")
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    W = GqaMoeWeights.from_params(cfg, params, dev)
    kv = KvCache(cfg, 64, dev)
    eng = GqaMoeEngine(cfg, W, kv, max_tokens=256, max_seqs=8)
    gen = Generator(eng, PagePool(64), max_pages_per_seq=8, max_seqs=8, prefill_chunk=128, use_graphs=use_graphs)
    return params, eng, gen


def glm_cfg() -> ModelConfig:
    """GLM-4.5 style layer: biased q / k / v, RoPE on the first half of every head, sigmoid routing under a correction
    bias, a shared expert."""
    return small_cfg().replace(name="glm4-moe-small", family="glm4_moe", qk_norm=False, rotary_dim=64, attention_bias=True,
                               scoring="sigmoid", router_bias=True, routed_scale=1.0, rms_eps=1e-5)


def swa_cfg() -> ModelConfig:
    """Hybrid stack: the second layer attends through a 48-token sliding window (shorter than a page and than the
    prompts), the first to everything."""
    c = small_cfg()
    return c.replace(name="swa-small", sliding_window=48, window_layers=tuple(i % 2 for i in range(c.num_layers)))


@pytest.mark.parametrize("use_graphs,family", [(False, "qwen3"), (True, "qwen3"), (False, "glm4"), (True, "glm4"), (False, "swa"), (True, "swa")])
def test_prefill_and_decode_match_oracle(use_graphs, family):
    from cuteafd_b200.models.gqa_moe import Batch
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.ref.model import KvState, RefDecoder
    cfg = {"qwen3": small_cfg, "glm4": glm_cfg, "swa": swa_cfg}[family]()
    params, eng, gen = build(cfg, use_graphs)
    ref = RefDecoder(cfg, params)
    g = torch.Generator().manual_seed(1)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (200, 77)]
    seqs, last, ref_kv, ref_logits = [], [], [], []
    with torch.no_grad():
        for p in prompts:
            s = gen.table.new()
            nxt = gen.prefill(s, p.tolist())          # chunked: 128 + rest
            kvs = KvState(cfg)
            rl = ref.forward(p, kvs)[-1]
            got = eng.logits[0].float().cpu()
            err = (got - rl).abs().max().item()
            assert err < 0.05 * max(rl.abs().max().item(), 1.0), err
            seqs.append(s); ref_kv.append(kvs); ref_logits.append(rl)
            last.append(int(rl.argmax()))             # teacher-force the oracle's token
        for step in range(6):
            new = gen.decode(seqs, last)
            torch.cuda.synchronize()
            assert K.read_status() == 0
            for i in range(len(seqs)):
                rl = ref.forward(torch.tensor([last[i]]), ref_kv[i])[-1]
                got = eng.logits[i].float().cpu()
                err = (got - rl).abs().max().item()
                assert err < 0.05 * max(rl.abs().max().item(), 1.0), (step, i, err)
                last[i] = int(rl.argmax())
    assert gen.h2d_bytes > 0 and gen.d2h_bytes > 0


@pytest.mark.parametrize("family", ["gqa", "mla"])
def test_mtp_depth_matches_oracle(family):
    """The multi-token-prediction depth (norms, split eh_proj, one decoder layer with its own K/V, shared head) after a
    prefill chunk and after a decode step."""
    from cuteafd_b200.models.gqa_moe import Batch
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    dev = torch.device("cuda:0")
    if family == "gqa":
        from cuteafd_b200.models.gqa_moe import GqaMoeEngine as Engine, GqaMoeWeights as Weights, KvCache as Cache
        cfg = small_cfg().replace(mtp_layers=1)
    else:
        from cuteafd_b200.models.mla_moe import LatentCache as Cache, MlaMoeEngine as Engine, MlaMoeWeights as Weights
        from tests.test_mla_gpu import _mla_cfg
        cfg = _mla_cfg().replace(mtp_layers=1)
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    eng = Engine(cfg, Weights.from_params(cfg, params, dev), Cache(cfg, 64, dev), max_tokens=256, max_seqs=8)
    gen = Generator(eng, PagePool(64), max_pages_per_seq=8, max_seqs=8, prefill_chunk=128, use_graphs=False)
    ref = RefDecoder(cfg, params)
    g = torch.Generator().manual_seed(3)
    n = 100
    p = torch.randint(0, cfg.vocab_size, (n,), generator=g)
    errs = []
    with torch.no_grad():
        s = gen.table.new()
        first = gen.prefill(s, p.tolist())
        b = gen.prefill_buf
        batch = Batch(b.tokens[1][:n], b.positions[1][:n], b.slots[1][:n], b.page_table[1].view(1, gen.max_pages),
                      b.seq_lens[1][:1], b.q_start[1][:2], n, True, None)
        nxt = torch.cat([p[1:], torch.tensor([first])])
        got = eng.mtp_forward(0, batch, nxt.to(torch.int32).to(dev)).float().cpu()
        kvs = KvState(cfg)
        h = ref.hidden_states(p, kvs)
        want, _ = ref.mtp_forward(0, h, nxt, torch.arange(n), kvs)
        for r in range(n):
            errs.append((got[r] - want[r]).abs().max().item() / max(want[r].abs().max().item(), 1.0))
        # one decode step: the depth sees (h of the new position, the token after it)
        tok2 = gen.decode([s], [first])[0]
        d = gen.decode_bufs[1]
        dbatch = Batch(d.tokens[1][:1], d.positions[1][:1], d.slots[1][:1], d.page_table[1].view(1, gen.max_pages),
                       d.seq_lens[1][:1], d.q_start[1][:2], 1, False, None)
        got2 = eng.mtp_forward(0, dbatch, torch.tensor([tok2], dtype=torch.int32, device=dev)).float().cpu()
        h2 = ref.hidden_states(torch.tensor([first]), kvs)
        want2, _ = ref.mtp_forward(0, h2, torch.tensor([tok2]), torch.tensor([n]), kvs)
        errs.append((got2[0] - want2[0]).abs().max().item() / max(want2[0].abs().max().item(), 1.0))
    torch.cuda.synchronize()
    assert K.read_status() == 0
    errs.sort()
    assert errs[len(errs) // 2] < 0.03 and errs[int(len(errs) * 0.9)] < 0.06 and errs[-1] < 0.3, errs[-10:]


def test_media_rows_through_the_engine_backend():
    """A prompt with media rows (ids above the vocabulary + embedding spans) prefilled in chunks by the engine
    backend gives the oracle's logits."""
    from cuteafd_b200.media.processor import MediaSpan, overrides_for
    from cuteafd_b200.ref.model import KvState, RefDecoder
    from cuteafd_b200.runtime.backends import EngineBackend
    cfg = small_cfg()
    params, eng, _ = build(cfg, False)
    be = EngineBackend(eng, 64, 8, prefill_chunk=64, max_decode_rows=4)
    g = torch.Generator().manual_seed(4)
    ids = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()
    emb = (torch.randn(70, cfg.hidden, generator=g) * 0.05).to(torch.bfloat16)
    span = MediaSpan(40, emb, b"k" * 16, "image")            # rows 40..109 cross two chunk boundaries
    for i in range(40, 110):
        ids[i] = cfg.vocab_size + 12345
    h, cached = be.open(ids)
    h.media = [span]
    assert cached == 0
    logits = None
    for c0 in range(0, len(ids), 64):
        logits = be.prefill(h, ids[c0:c0 + 64], c0 + 64 >= len(ids))
    ref = RefDecoder(cfg, params)
    rl = ref.forward(torch.tensor(ids), KvState(cfg), overrides_for([span], 0, len(ids)))[-1]
    err = (logits[0] - rl).abs().max().item()
    assert err < 0.05 * max(rl.abs().max().item(), 1.0), err
    with pytest.raises(ValueError):
        h2, _ = be.open(ids)
        be.prefill(h2, ids[:64], False)                      # media ids without their spans


def test_vision_tower_on_the_gpu_matches_cpu():
    """bf16 tower with its projections on the tcgen05 GEMM against the fp32 CPU tower."""
    from cuteafd_b200.media import VisionTower, VisionTowerConfig, preprocess_image
    cfg = VisionTowerConfig(width=256, depth=2, heads=4, mlp=512, out_hidden=512)
    w = {k: v.to(torch.bfloat16).float() for k, v in VisionTower.random_weights(cfg, seed=3, std=0.05).items()}
    px = torch.randint(0, 255, (120, 200, 3), generator=torch.Generator().manual_seed(0), dtype=torch.uint8)
    patches, grid = preprocess_image(px)
    ref = VisionTower(cfg, w, "cpu").forward(patches, grid)
    got = VisionTower(cfg, w, "cuda:0").forward(patches, grid).float().cpu()
    assert got.shape == ref.shape
    err = (got - ref).abs().max().item() / max(ref.abs().max().item(), 1e-6)
    assert err < 0.05, err


def test_decode_graph_bank_and_prewarm(tmp_path):
    """The serving backend replays one CUDA graph per step geometry: same tokens as the eager path, a geometry is
    captured on its second sight, a saved prewarm list captures before traffic."""
    import json
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = small_cfg()
    g = torch.Generator().manual_seed(7)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (70, 33, 90)]

    def run(use_graphs, prewarm=None):
        _, eng, _ = build(cfg, False)
        be = EngineBackend(eng, 64, 8, prefill_chunk=64, max_decode_rows=4, use_graphs=use_graphs)
        if prewarm:
            assert be.prewarm(prewarm) == len(prewarm)
        sched = Scheduler(be, max_active=4)
        reqs = [Request(prompt=list(p), max_tokens=12, speculation=False) for p in prompts]
        for r in reqs:
            sched.submit(r)
        toks = [[] for _ in reqs]
        done = 0
        for _ in range(400):
            sched.step()
            for i, r in enumerate(reqs):
                while not r.events.empty():
                    ev = r.events.get()
                    if ev[0] == "tokens":
                        toks[i] += ev[1]
                    elif ev[0] in ("done", "error"):
                        assert ev[0] == "done", ev
                        done += 1
            if done == len(reqs):
                break
        assert done == len(reqs)
        torch.cuda.synchronize()
        assert K.read_status() == 0
        return toks, be

    eager, be0 = run(False)
    graphs, be1 = run(True)
    assert eager == graphs
    assert be0.graph_stats["replays"] == 0 and be1.graph_stats["replays"] > 0 and be1.graph_stats["captures"] >= 1
    path = str(tmp_path / "prewarm.json")
    keys = be1.save_prewarm(path, top=2)
    assert json.load(open(path))["geometries"] == keys and len(keys) >= 1
    warm, be2 = run(True, prewarm=keys)
    assert warm == eager
    assert be2.graph_stats["captures"] >= len(keys) and be2.graph_stats["eager"] < be1.graph_stats["eager"] + 1
    # byte-measured arena: the file carries what the captures made the allocator reserve, and the planner can read it
    doc = json.load(open(path))
    res = be1.graph_reserve()
    assert doc["reserve_base_bytes"] == res["reserve_base_bytes"] >= 0 and doc["reserve_extra_bytes"] == res["reserve_extra_bytes"]
    assert set(doc["graph_bytes"]) == {",".join(map(str, k)) for k in be1.graph_bytes}
    from cuteafd_b200.cli import graph_reserve_of
    assert graph_reserve_of(path)[0] == doc["reserve_base_bytes"] + doc["reserve_extra_bytes"]
    # a byte budget smaller than one capture: at most one graph is ever held, nothing breaks, tokens are the same
    _, eng3, _ = build(small_cfg(), False)
    from cuteafd_b200.runtime.backends import EngineBackend
    be3 = EngineBackend(eng3, 64, 8, prefill_chunk=64, max_decode_rows=4, use_graphs=True)
    be3.graph_budget_bytes = 1
    be3.graph_bytes[(0, 0, 0)] = 1 << 20                    # pretend an earlier capture took 1 MiB: the next guess is over budget
    assert be3.prewarm([[1, 1, 1], [2, 2, 1]]) == 2 and len(be3.graphs) == 0 and be3.graph_stats["refused"] == 2


def test_prompt_packing_on_the_engine():
    """Chunks of several prompts in one engine step (multi-sequence prefill batch) give the tokens of serving the
    prompts one at a time."""
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = small_cfg()
    g = torch.Generator().manual_seed(11)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (30, 70, 9, 100)]

    def serve(max_active):
        _, eng, _ = build(cfg, False)
        be = EngineBackend(eng, 64, 8, prefill_chunk=128, max_decode_rows=4, use_graphs=False)
        sched = Scheduler(be, max_active=max_active)
        reqs = [Request(prompt=list(p), max_tokens=6, speculation=False) for p in prompts]
        for r in reqs:
            sched.submit(r)
        out = [[] for _ in reqs]
        for _ in range(400):
            sched.step()
            for i, r in enumerate(reqs):
                while not r.events.empty():
                    ev = r.events.get()
                    if ev[0] == "tokens":
                        out[i] += ev[1]
                    assert ev[0] != "error", ev
            if sched.stats.finished == len(reqs):
                break
        torch.cuda.synchronize()
        assert K.read_status() == 0 and sched.stats.finished == len(reqs)
        return out, sched.stats.packed_steps
    alone, p1 = serve(1)
    packed, p4 = serve(4)
    assert p1 == 0 and p4 >= 1
    # batched and single-sequence kernels round alike here (same tiles per sequence); allow a late divergence only
    same = sum(a[:3] == b[:3] for a, b in zip(alone, packed))
    assert same == len(prompts), (alone, packed)


def test_probe_scoring_and_state_hash_on_the_engine():
    """Probe fields on the CUDA backend: teacher-forced scoring rows agree with the oracle's teacher-forced log-probs, and
    the state hash of a prompt is the same cold and through the prefix cache (pages differ, bytes do not)."""
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.ref.model import KvState, RefDecoder
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler, collect
    cfg = small_cfg()
    params, eng, _ = build(cfg, False)
    be = EngineBackend(eng, 64, 8, prefill_chunk=64, max_decode_rows=8, use_graphs=False)
    sched = Scheduler(be, max_active=2)
    g = torch.Generator().manual_seed(5)
    ids = torch.randint(0, cfg.vocab_size, (150,), generator=g).tolist()

    def run(req):
        sched.submit(req)
        for _ in range(300):
            sched.step()
            if not sched.pending and not sched.prefilling and not sched.decoding:
                break
        return collect(req, timeout=5)
    out = run(Request(prompt=list(ids), max_tokens=4, score_from=100, verify_rows=5, top_logprobs=1))
    assert out["error"] is None and out["tokens"] == []
    rows = out["usage"]["score_rows"]
    assert [r["position"] for r in rows] == list(range(100, 150))
    with torch.no_grad():
        lp = torch.log_softmax(RefDecoder(cfg, params).forward(torch.tensor(ids), KvState(cfg)).float(), -1)
    errs = sorted(abs(r["logprob"] - float(lp[r["position"] - 1, r["token"]])) for r in rows)
    assert errs[len(errs) // 2] < 0.05 and errs[-1] < 0.5, errs
    a = run(Request(prompt=list(ids), max_tokens=3, cold=True, record_state=True, speculation=False))
    b = run(Request(prompt=list(ids), max_tokens=3, record_state=True, speculation=False))
    ha, hb = a["usage"]["state_hashes"], b["usage"]["state_hashes"]
    assert b["usage"]["cached_tokens"] >= 64 and [h["frontier"] for h in ha] == ["prompt", "turn"]
    assert ha[0]["hash"] == hb[0]["hash"] and ha[0]["hash"] != ha[1]["hash"]
    torch.cuda.synchronize()
    assert K.read_status() == 0


def test_host_tier_evict_and_restore_on_the_engine():
    """Pinned-host tier behind the device prefix cache: snapshots evicted by other traffic are copied out on the side
    stream and copied back on a later hit; the request served from the host tier emits the same tokens and the same
    logit row hashes as when the device tier served the same prefix."""
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler
    cfg = small_cfg()
    _, eng, _ = build(cfg, False)            # 64 KV pages
    be = EngineBackend(eng, 40, 12, prefill_chunk=128, max_decode_rows=4, use_graphs=False,
                       host_cache_bytes=64 * eng.kv.bytes_per_page())
    assert be.tier is not None
    sched = Scheduler(be, max_active=1)

    def serve(prompt, n):
        r = Request(prompt=list(prompt), max_tokens=n, speculation=False, record_rows=True)
        sched.submit(r)
        toks, usage, hashes = [], None, None
        for _ in range(600):
            sched.step()
            while not r.events.empty():
                ev = r.events.get()
                if ev[0] == "tokens":
                    toks += ev[1]
                elif ev[0] == "done":
                    usage, hashes = ev[2], ev[3]
                else:
                    raise AssertionError(ev)
            if usage is not None:
                break
        assert usage is not None
        return toks, usage, hashes

    g = torch.Generator().manual_seed(31)
    prompt = torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist()
    cold = serve(prompt, 6)
    dev_hit = serve(prompt, 6)
    assert dev_hit[1]["cached_tokens"] >= 512 and dev_hit[0] == cold[0]
    for _ in range(4):
        serve(torch.randint(0, cfg.vocab_size, (600,), generator=g).tolist(), 2)
    assert be.prefix.stats.spilled >= 1 and be.tier.host.stats.stored >= 1
    host_hit = serve(prompt, 6)
    torch.cuda.synchronize()
    assert K.read_status() == 0
    assert be.prefix.stats.restored >= 1 and host_hit[1]["cached_tokens"] >= 512
    assert host_hit[0] == dev_hit[0] and host_hit[2] == dev_hit[2]
    be.tier.host.check_invariants()


@pytest.mark.parametrize("fmt", ["fp8_block128", "mxfp4", "nvfp4"])
def test_snapshot_served_in_its_stored_format(fmt, tmp_path):
    """A random snapshot whose routed experts are E4M3 block-scaled / MXFP4 / NVFP4 is loaded without decoding them
    (the engine holds the stored bytes) and its logits match the oracle that decodes the same snapshot."""
    from cuteafd_b200.loader.load import load_engine, load_params
    from cuteafd_b200.loader.snapshot import write_random_snapshot
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.ref.model import KvState, RefDecoder
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    path = write_random_snapshot(small_cfg(), str(tmp_path / "snap"), fmt=fmt, seed=5)
    dev = torch.device("cuda:0")
    cfg, eng = load_engine(path, dev, 64, 256, 8)
    assert eng.W.expert_format == {"fp8_block128": "fp8"}.get(fmt, fmt)
    stored = eng.W.layers[1].w_gate
    assert isinstance(stored, tuple) and stored[0].dtype in (torch.float8_e4m3fn, torch.uint8)
    _, params = load_params(path)
    ref = RefDecoder(cfg, params)
    gen = Generator(eng, PagePool(64), max_pages_per_seq=8, max_seqs=8, prefill_chunk=128, use_graphs=False)
    g = torch.Generator().manual_seed(2)
    p = torch.randint(0, cfg.vocab_size, (150,), generator=g)
    errs = []
    with torch.no_grad():
        s = gen.table.new()
        gen.prefill(s, p.tolist())
        kvs = KvState(cfg)
        rl = ref.forward(p, kvs)[-1]
        errs.append((eng.logits[0].float().cpu() - rl).abs().max().item() / max(rl.abs().max().item(), 1.0))
        last = int(rl.argmax())
        for _ in range(3):
            gen.decode([s], [last])
            rl = ref.forward(torch.tensor([last]), kvs)[-1]
            errs.append((eng.logits[0].float().cpu() - rl).abs().max().item() / max(rl.abs().max().item(), 1.0))
            last = int(rl.argmax())
    torch.cuda.synchronize()
    assert K.read_status() == 0
    assert max(errs) < 0.06, errs


def test_host_resident_embedding_table(tmp_path):
    """``--embedding-placement host``: the embedding table stays memory-mapped in the snapshot, every step's rows are
    gathered and staged; replies equal the ones with the table on the GPU, eagerly and through captured decode graphs."""
    from cuteafd_b200.loader.load import host_embedding_table, load_engine
    from cuteafd_b200.loader.snapshot import write_random_snapshot
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler, collect
    snap = write_random_snapshot(small_cfg(), str(tmp_path / "snap"), fmt="bf16", seed=5)
    g = torch.Generator().manual_seed(2)
    prompts = [torch.randint(0, small_cfg().vocab_size, (n,), generator=g).tolist() for n in (150, 40, 9)]

    def serve(host: bool, graphs: bool):
        cfg, eng = load_engine(snap, torch.device("cuda:0"), 64, 256, 8)
        table = host_embedding_table(snap) if host else None
        if host:
            eng.W.embed = None
        be = EngineBackend(eng, 64, 8, prefill_chunk=64, max_decode_rows=4, use_graphs=graphs, host_embedding=table)
        sched = Scheduler(be, max_active=4)
        reqs = [sched.submit(Request(prompt=list(p), max_tokens=8, speculation=False)) for p in prompts]
        for _ in range(400):
            sched.step()
            if sched.stats.finished == len(reqs):
                break
        outs = [collect(r, timeout=5) for r in reqs]
        assert all(o["error"] is None for o in outs), outs
        torch.cuda.synchronize()
        assert K.read_status() == 0
        return [o["tokens"] for o in outs], table
    want, _ = serve(False, False)
    got, table = serve(True, False)
    assert got == want and table.stats.rows >= sum(len(p) for p in prompts) and table.stats.prefetch_hits >= 0
    got_g, _ = serve(True, True)
    assert got_g == want


@pytest.mark.parametrize("parallel", [False, True])
def test_draft_model_on_the_gpu(parallel):
    """A draft model that is a CUDA engine (here: a second instance of the target's own weights): replies equal the
    non-speculative ones; the sequential drafter's proposals are what the target picks (nearly all accepted), the block
    drafter produces its block in one pass per round."""
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.backends import EngineBackend
    from cuteafd_b200.runtime.scheduler import Request, Scheduler, collect
    from cuteafd_b200.runtime.speculation import ModelDrafter
    cfg = small_cfg()
    g = torch.Generator().manual_seed(21)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist() for n in (90, 33)]

    def serve(drafter):
        _, eng, _ = build(cfg, False)
        be = EngineBackend(eng, 64, 8, prefill_chunk=64, max_decode_rows=4, use_graphs=False)
        kw = dict(drafter=drafter, draft_control="always") if drafter is not None else {}
        sched = Scheduler(be, max_active=2, **kw)
        reqs = [sched.submit(Request(prompt=list(p), max_tokens=16, speculation=drafter is not None)) for p in prompts]
        for _ in range(600):
            sched.step()
            if sched.stats.finished == len(reqs):
                break
        outs = [collect(r, timeout=5) for r in reqs]
        assert all(o["error"] is None for o in outs), outs
        torch.cuda.synchronize()
        assert K.read_status() == 0
        return outs
    base = serve(None)
    _, draft_eng, _ = build(cfg, False)                      # same seed: the target's own weights
    drafter = ModelDrafter.from_engine(draft_eng, 64, 8, block=3, parallel=parallel)
    outs = serve(drafter)
    prop = sum(o["usage"]["speculation"]["proposed"] for o in outs)
    acc = sum(o["usage"]["speculation"]["accepted"] for o in outs)
    cyc = sum(o["usage"]["speculation"]["cycles"] for o in outs)
    same = sum(a["tokens"][:6] == b["tokens"][:6] for a, b in zip(outs, base))
    assert same == len(prompts), ([o["tokens"] for o in outs], [o["tokens"] for o in base])
    assert prop > 0 and drafter.model.steps > 0 and drafter.state == {}
    if parallel:
        assert drafter.passes <= cyc and acc >= cyc // 3           # position 1 of most blocks is the target's own pick
    else:
        assert acc >= 0.7 * prop                                   # the same model in another step shape: near-ties aside


def test_step_staging_is_not_overwritten_before_its_copy_ran():
    """The GPU can be a whole prompt chunk behind the host: what ``upload`` sends must be the values at the call, not
    what the caller writes into the staging views for the next chunk while the copy is still queued."""
    from cuteafd_b200.runtime.generate import StepBuffers
    dev = torch.device("cuda:0")
    b = StepBuffers(256, 1, 8, dev)
    busy = torch.randn(4096, 4096, device=dev)
    torch.cuda.synchronize()
    for _ in range(60):                              # tens of milliseconds of queued work in front of the copies
        busy = busy @ busy * 1e-3
    seen = []
    for chunk in range(4):
        b.tokens[0][:] = chunk + 1
        b.upload()
        seen.append(b.tokens[1].clone())             # stream-ordered after this chunk's copy
    b.tokens[0][:] = 99
    torch.cuda.synchronize()
    assert [int(t[0]) for t in seen] == [1, 2, 3, 4] and all(bool((t == t[0]).all()) for t in seen)
