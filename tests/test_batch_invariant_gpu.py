"""Batch-invariant decode: with fixed kv splits a row's logits are the same bits whether the sequence decodes alone or
among other sequences of any length, up to the decode capacity of 64 rows (the reference's contract:
REPORT-kernel-210.md:14-66, native/CMakeLists.txt:108-109)."""
import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.fixture
def fixed_splits():
    from cuteafd_b200.ops import kernels as K
    K.set_fixed_kv_split(1024)
    try:
        yield K
    finally:
        K.set_fixed_kv_split(0)


def _engine(family, dev):
    from cuteafd_b200.ref.model import init_weights
    if family == "gqa":
        from cuteafd_b200.models.gqa_moe import GqaMoeEngine as Engine, GqaMoeWeights as Weights, KvCache as Cache
        from tests.test_engine_gpu import small_cfg
        cfg = small_cfg()
    else:
        from cuteafd_b200.models.mla_moe import LatentCache as Cache, MlaMoeEngine as Engine, MlaMoeWeights as Weights
        from tests.test_mla_gpu import _mla_cfg
        cfg = _mla_cfg()
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    eng = Engine(cfg, Weights.from_params(cfg, params, dev), Cache(cfg, 640, dev), max_tokens=256, max_seqs=64)
    return cfg, eng


@pytest.mark.parametrize("family,use_graphs", [("gqa", False), ("gqa", True), ("mla", False)])
def test_a_rows_bits_do_not_depend_on_the_step(fixed_splits, family, use_graphs):
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    K = fixed_splits
    dev = torch.device("cuda:0")
    cfg, eng = _engine(family, dev)
    assert eng.fixed_kv_split == 1024
    g = torch.Generator().manual_seed(5)
    target = torch.randint(0, cfg.vocab_size, (1500,), generator=g).tolist()        # spans two kv splits
    forced = [5, 17, 99, 3]

    def run(others: list[int], at: int):
        gen = Generator(eng, PagePool(640), max_pages_per_seq=40, max_seqs=64, prefill_chunk=128, use_graphs=use_graphs)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=torch.Generator().manual_seed(100 + n)).tolist() for n in others]
        prompts.insert(at, target)
        seqs = []
        with torch.no_grad():
            for p in prompts:
                s = gen.table.new()
                gen.prefill(s, p)
                seqs.append(s)
            rows = []
            for step, tok in enumerate(forced):
                gen.decode(seqs, [tok if i == at else (7 * i + step) % cfg.vocab_size for i in range(len(seqs))])
                torch.cuda.synchronize()
                assert K.read_status() == 0
                rows.append(eng.logits[at].clone())
        return rows

    alone = run([], 0)
    among8 = run([50, 2000, 700, 64, 1, 1029, 333], 3)
    among40 = run([20 + 3 * i for i in range(39)], 17)
    diffs = [(name, step, (alone[step].float() - other[step].float()).abs().max().item())
             for name, other in (("among 8", among8), ("among 40", among40)) for step in range(len(forced))
             if not torch.equal(alone[step], other[step])]
    assert not diffs, diffs
