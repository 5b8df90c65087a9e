"""The placement solver over every preset and inventory: an accepted plan never oversubscribes a GPU, its expert ranges
tile the expert ids exactly once, the pool is whole pages and at least the minimum, the deployment document passes the
launcher's own validation, and a smaller memory cap never turns a refusal into an acceptance."""
import pytest
from hypothesis import given, settings
from hypothesis import strategies as st

from cuteafd_b200.config import PRESETS
from cuteafd_b200.planner.solver import GIB, PlacementRequest, solve


@settings(max_examples=120)
@given(name=st.sampled_from(sorted(PRESETS)), gpus=st.integers(1, 8), cap=st.sampled_from([40, 80, 141, 179]),
       att=st.sampled_from([None, 1, 2, 4]), exp=st.sampled_from([None, 0, 1, 3, 6, 7]), ctx=st.sampled_from([8192, 131072]),
       fmt=st.sampled_from([None, "fp8_block128", "nvfp4"]))
def test_accepted_plans_fit_and_tile(name, gpus, cap, att, exp, ctx, fmt):
    cfg = PRESETS[name]()
    if not cfg.num_experts and exp not in (None, 0):
        exp = 0
    req = PlacementRequest(cfg, gpus=gpus, gpu_memory_cap=cap * GIB, attention_ranks=att, expert_ranks=exp, max_context_tokens=ctx,
                           expert_format=fmt if cfg.num_experts else None)
    p = solve(req)
    if not p.ok:
        assert p.reason
        bigger = solve(PlacementRequest(cfg, gpus=gpus, gpu_memory_cap=(cap // 2) * GIB, attention_ranks=att, expert_ranks=exp,
                                        max_context_tokens=ctx, expert_format=fmt if cfg.num_experts else None))
        assert not bigger.ok                                   # half the memory does not help
        return
    used = [g for g in p.devices if g.role != "idle"]
    assert len(used) == p.attention_ranks * p.pipeline_stages + p.expert_ranks <= gpus
    assert all(g.free >= 0 and g.used <= cap * GIB for g in used)
    assert p.kv_pool_tokens % 64 == 0 and p.kv_pool_tokens >= min(req.pool_tokens_min, req.pool_tokens_target)
    if cfg.num_experts:
        spans = sorted(p.expert_ranges)
        assert spans[0][0] == 0 and spans[-1][1] == cfg.num_experts and all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
    assert p.notes and (p.engine in ("single", "afd", "tp", "pp", ""))


@pytest.mark.parametrize("name", sorted(PRESETS))
def test_deployment_documents_of_served_layouts_pass_the_launcher(name):
    from cuteafd_b200 import launch as LA
    from cuteafd_b200.planner import plan as P
    from cuteafd_b200.planner.solver import HTTP_ENGINES
    rep = P.plan(name, layout=True, gpus=8)
    if not (rep.placement and rep.placement.ok):
        pytest.skip(f"{name} does not fit eight GPUs in its stored format")
    doc = P.deployment(rep)
    LA.validate(doc)
    assert doc["world_size"] == len(doc["ranks"]) and doc["engine"] == rep.placement.engine
    if rep.placement.engine in HTTP_ENGINES:
        assert doc["ranks"][0]["role"].startswith("attention")
