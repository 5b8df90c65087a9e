"""Weight arena and memory ledger (host memory; the same code runs with a CUDA device)."""
import json

import pytest
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.loader import load, snapshot
from cuteafd_b200.runtime.arena import ALIGN, ArenaError, WeightArena
from cuteafd_b200.utils.memory_ledger import MemoryLedger


def test_arena_views_are_aligned_and_disjoint():
    led = MemoryLedger(probe=lambda d: (0, 0))
    ar = WeightArena("cpu", "t", led)
    ar.reserve("a", (3, 5), torch.bfloat16)
    ar.reserve("b", (7,), torch.float32)
    ar.reserve("c", (2, 2, 2), torch.uint8)
    with pytest.raises(ArenaError):
        ar.reserve("a", (1,), torch.uint8)
    with pytest.raises(ArenaError):
        ar.view("a")
    ar.allocate()
    ptrs = {n: ar.view(n).data_ptr() for n in "abc"}
    assert all(p % ALIGN == 0 for p in ptrs.values())
    ar.fill("a", torch.ones(3, 5, dtype=torch.bfloat16))
    ar.fill_rows("b", 0, torch.arange(4, dtype=torch.float32))
    assert ar.missing() == ["b", "c"]
    ar.fill_rows("b", 4, torch.arange(3, dtype=torch.float32))
    ar.fill("c", torch.full((2, 2, 2), 9, dtype=torch.uint8))
    assert ar.missing() == []
    assert ar.view("a").sum() == 15 and ar.view("b").tolist() == [0, 1, 2, 3, 0, 1, 2] and ar.view("c").min() == 9
    with pytest.raises(ArenaError):
        ar.fill_rows("b", 5, torch.zeros(3))
    with pytest.raises(ArenaError):
        ar.fill("a", torch.zeros(5, 3, dtype=torch.bfloat16))
    d = ar.describe()
    assert d["tensors"] == 3 and d["bytes"] == 3 * ALIGN and d["padding"] == 3 * ALIGN - (30 + 28 + 8)
    assert led.report()["by_kind"] == {"weights": 3 * ALIGN + ALIGN}
    ar.release()
    assert led.total() == 0


def test_arena_refuses_a_plan_that_does_not_fit():
    ar = WeightArena("cpu", "big", MemoryLedger(probe=lambda d: (0, 0)))
    ar.reserve("w", (1024, 1024), torch.bfloat16)
    with pytest.raises(ArenaError, match="do not fit"):
        ar.check_fits(free_bytes=1 << 20)
    with pytest.raises(ArenaError, match="reserve"):
        ar.check_fits(free_bytes=3 << 20, reserve_bytes=2 << 20)
    ar.check_fits(free_bytes=3 << 20)


def test_ledger_tree_reconcile_and_failure_spool(tmp_path):
    led = MemoryLedger(probe=lambda d: (60 << 20, 100 << 20))

    class Holder:
        __module__ = "cuteafd_b200.fake"

    h = Holder()
    base = torch.zeros(1 << 20, dtype=torch.uint8)
    h.a, h.view_of_a, h.more = base, base[:10], {"x": [torch.zeros(256, dtype=torch.float32)]}
    Holder.__module__ = "cuteafd_b200.fake"
    got = led.tag_tree("kv", "engine", h)
    assert got == (1 << 20) + 1024                       # the view shares storage: counted once
    from cuteafd_b200.models.gqa_moe import LayerWeights                  # a __slots__ class: no __dict__ to walk
    L = LayerWeights()
    L.wo = torch.zeros(512, dtype=torch.float32)
    assert led.tag_tree("weights", "layer", [L]) == 2048
    led.release("weights", "layer")
    led.tag("graphs", "bank", 5 << 20, "cpu")
    rec = led.reconcile()["cpu"]
    assert rec["used"] == 40 << 20 and rec["untracked"] == (40 << 20) - led.total("cpu")
    spool = str(tmp_path / "spool" / "memory_failures.jsonl")
    led.open_spool(spool)
    with pytest.raises(RuntimeError):
        with led.guard("prefill workspace"):
            raise RuntimeError("CUDA out of memory. Tried to allocate 20.00 GiB")
    with pytest.raises(RuntimeError):
        with led.guard("other"):
            raise RuntimeError("shape mismatch")       # not a memory failure: nothing recorded
    lines = open(spool).read().splitlines()
    assert len(lines) == 1 and json.loads(lines[0])["what"] == "prefill workspace"
    assert json.loads(lines[0])["by_kind"]["graphs"] == 5 << 20
    assert any("tracked" in l for l in led.lines())
    led.release("kv", "engine")
    assert led.report()["by_kind"] == {"graphs": 5 << 20}


def test_engine_weights_load_into_one_arena(tmp_path):
    """The arena loader gives the engine the same tensors as the dictionary path, as views of one buffer."""
    from cuteafd_b200.models.gqa_moe import GqaMoeWeights
    cfg = tiny_moe().replace(family="qwen3_moe", attention="gqa", num_heads=2, num_kv_heads=2, head_dim=64, hidden=128,
                             expert_ffn=128, dense_ffn=128, num_experts=4, top_k=2, vocab_size=256, num_shared_experts=1,
                             scoring="softmax", qk_norm=True)
    src = snapshot.write_random_snapshot(cfg, str(tmp_path / "s"), fmt="fp8_block128", seed=4)
    cfg2, W = load.load_gqa_engine_weights(src, torch.device("cpu"))
    _, params = load.load_params(src, dtype=torch.bfloat16)
    ref = GqaMoeWeights.from_params(cfg2, params, torch.device("cpu"))
    assert torch.equal(W.embed, ref.embed) and torch.equal(W.final_norm, ref.final_norm)
    for a, b in zip(W.layers, ref.layers):
        for name in ("ln1", "ln2", "wqkv", "wo", "q_norm", "k_norm", "router", "w_gate", "w_up", "w_down", "s_gate", "s_up",
                     "s_down", "d_gate", "d_up", "d_down"):
            x, y = getattr(a, name, None), getattr(b, name, None)
            assert (x is None) == (y is None), name
            if x is not None:
                assert x.shape == y.shape and torch.equal(x, y), name
                assert x.data_ptr() % ALIGN == 0 and x.is_contiguous()
    lo, hi = W.arena.buf.data_ptr(), W.arena.buf.data_ptr() + W.arena.size
    assert all(lo <= getattr(L, "wqkv").data_ptr() < hi for L in W.layers)
    # experts of a range only (an expert rank's share)
    _, We = load.load_gqa_engine_weights(src, torch.device("cpu"), expert_range=(1, 3))
    moe = next(i for i in range(cfg2.num_layers) if cfg2.is_moe_layer(i))
    assert We.layers[moe].w_up.shape[0] == 2 and torch.equal(We.layers[moe].w_up, ref.layers[moe].w_up[1:3])
