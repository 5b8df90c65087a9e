"""The one-launch decode step (csrc/decode_step.cu) against the CPU oracle and against the per-op kernels."""
import pytest
import torch

from cuteafd_b200.config import ModelConfig

pytestmark = pytest.mark.gpu


@pytest.fixture(autouse=True)
def _fused_on(monkeypatch):
    monkeypatch.setenv("CAFD_FUSED_DECODE", "1")      # the one-launch step is opt-in


def cfg_small() -> ModelConfig:
    return ModelConfig(name="gqa-moe-fused-small", family="qwen3_moe", vocab_size=2048, num_layers=3, hidden=512,
                       attention="gqa", num_heads=8, num_kv_heads=2, head_dim=128, qk_norm=True, rope_theta=1e6,
                       rope_interleaved=False, dense_ffn=1024, first_dense_layers=0, num_experts=16, expert_ffn=256,
                       top_k=4, scoring="softmax", num_shared_experts=0)


def cfg_wide() -> ModelConfig:
    """Qwen3-30B-A3B widths (hidden 2048, 32 / 4 heads: o projection in two K passes, expert FFN 768), one layer."""
    return ModelConfig(name="gqa-moe-fused-wide", family="qwen3_moe", vocab_size=1024, num_layers=1, hidden=2048,
                       attention="gqa", num_heads=32, num_kv_heads=4, head_dim=128, qk_norm=True, rope_theta=1e6,
                       rope_interleaved=False, dense_ffn=1024, first_dense_layers=0, num_experts=8, expert_ffn=768,
                       top_k=8, scoring="softmax", num_shared_experts=0)


def build(cfg, use_graphs, pages=96, max_seqs=32):
    from cuteafd_b200.models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
    from cuteafd_b200.ref.model import init_weights
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    dev = torch.device("cuda:0")
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    W = GqaMoeWeights.from_params(cfg, params, dev)
    kv = KvCache(cfg, pages, dev)
    eng = GqaMoeEngine(cfg, W, kv, max_tokens=256, max_seqs=max_seqs)
    gen = Generator(eng, PagePool(pages), max_pages_per_seq=8, max_seqs=max_seqs, prefill_chunk=128, use_graphs=use_graphs)
    return params, eng, gen


def _close(got, want, tol=0.03):
    err = (got - want).abs().max().item()
    assert err < tol * max(want.abs().max().item(), 1.0), err


@pytest.mark.parametrize("which,use_graphs", [("small", False), ("small", True), ("wide", False)])
def test_fused_decode_matches_oracle(which, use_graphs):
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.ops.decode_step import FusedDecodeStep
    from cuteafd_b200.ref.model import KvState, RefDecoder
    cfg = cfg_small() if which == "small" else cfg_wide()
    assert FusedDecodeStep.supports(cfg)
    params, eng, gen = build(cfg, use_graphs)
    ref = RefDecoder(cfg, params)
    g = torch.Generator().manual_seed(1)
    lens = (200, 77, 5, 126) if which == "small" else (70, 9)
    prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in lens]
    seqs, last, ref_kv = [], [], []
    with torch.no_grad():
        for p in prompts:
            s = gen.table.new()
            gen.prefill(s, p.tolist())
            kvs = KvState(cfg)
            rl = ref.forward(p, kvs)[-1]
            seqs.append(s); ref_kv.append(kvs)
            last.append(int(rl.argmax()))
        for step in range(5):                      # sequence 3 crosses a page boundary (126 -> 131)
            new = gen.decode(seqs, last)
            torch.cuda.synchronize()
            assert K.read_status() == 0
            assert eng.fused is not None and eng.fused.launches > 0, "the fused step did not run"
            for i in range(len(seqs)):
                rl = ref.forward(torch.tensor([last[i]]), ref_kv[i])[-1]
                got = eng.logits[i].float().cpu()
                _close(got, rl)
                assert new[i] == int(got.argmax()), (step, i)       # in-kernel selection = argmax of its own logits
                last[i] = int(rl.argmax())


@pytest.mark.parametrize("rows", [1, 9, 17, 32])
def test_fused_equals_per_op_kernels(rows):
    """Same weights, same cache contents: the fused step and the launch-per-op path give the same logits (up to the
    different summation order) for every column-tile count, and the fused step is bitwise reproducible."""
    from cuteafd_b200.models.gqa_moe import Batch
    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.runtime.generate import StepBuffers
    from cuteafd_b200.runtime.paged import PAGE
    cfg = cfg_small()
    params, eng, gen = build(cfg, False, pages=200)
    g = torch.Generator().manual_seed(rows)
    seqs, toks = [], []
    for i in range(rows):
        s = gen.table.new()
        n = 3 + (i * 37) % 150
        toks.append(gen.prefill(s, torch.randint(0, cfg.vocab_size, (n,), generator=g).tolist()))
        seqs.append(s)
    b = StepBuffers(rows, rows, gen.max_pages, gen.device)
    pt = b.page_table[0].view(rows, gen.max_pages)
    for i, (s, tok) in enumerate(zip(seqs, toks)):
        gen.table.reserve(s, s.kv_len + 4)
        b.tokens[0][i], b.positions[0][i] = tok, s.kv_len
        b.slots[0][i] = s.pages[s.kv_len // PAGE] * PAGE + s.kv_len % PAGE
        pt[i, :len(s.pages)] = torch.tensor(s.pages, dtype=torch.int32)
        b.seq_lens[0][i], b.q_start[0][i] = s.kv_len + 1, i
    b.q_start[0][rows] = rows
    b.upload()
    batch = Batch(b.tokens[1][:rows], b.positions[1][:rows], b.slots[1][:rows], b.page_table[1].view(rows, gen.max_pages),
                  b.seq_lens[1][:rows], b.q_start[1][:rows + 1], 1, False, None)
    fused = eng.forward(batch).float().cpu().clone()
    picked = eng.greedy(eng.logits[:rows]).cpu().clone()
    assert eng.fused is not None and eng.fused.launches == 1
    again = eng.forward(batch).float().cpu().clone()
    assert torch.equal(fused, again)
    f, eng.fused = eng.fused, None                  # same step through the per-op kernels (writes the same K/V again)
    plain = eng.forward(batch).float().cpu().clone()
    eng.fused = f
    torch.cuda.synchronize()
    assert K.read_status() == 0
    _close(fused, plain, tol=0.02)
    assert torch.equal(picked.long(), fused.argmax(dim=1))
    # device-side advance: tokens, positions, lengths and slots move to the next step
    pos0 = batch.positions.cpu().clone()
    out = eng.decode_step(batch, advance=True).cpu()
    torch.cuda.synchronize()
    assert torch.equal(batch.tokens.cpu(), out) and torch.equal(batch.positions.cpu(), pos0 + 1)
    assert torch.equal(batch.seq_lens.cpu(), pos0 + 2)
    want_slots = torch.tensor([s.pages[(int(p) + 1) // PAGE] * PAGE + (int(p) + 1) % PAGE for s, p in zip(seqs, pos0)], dtype=torch.int32)
    assert torch.equal(batch.slots.cpu(), want_slots)
