"""Placement planner and the `cuteafd plan` command (CPU only)."""
import json

import pytest

from cuteafd_b200 import deepseek_v3, qwen3_30b_a3b, tiny_moe
from cuteafd_b200.cli import load_config_file, main
from cuteafd_b200.planner import plan as P
from cuteafd_b200.planner import solver


def test_deepseek_fp8_on_eight_gpus_fits_and_splits_experts():
    rep = P.plan("deepseek-v3", layout=True, gpus=8, attention_ranks=2, expert_ranks=6)
    p = rep.placement
    assert p.ok and p.layout == "attention tp2 + experts ep6"
    assert [hi - lo for lo, hi in p.expert_ranges] == [43, 43, 43, 43, 42, 42]
    assert p.expert_ranges[0][0] == 0 and p.expert_ranges[-1][1] == 256
    assert p.kv_pool_tokens == 2_097_152 and p.kv_bytes_per_token == 656 * 61
    for g in p.devices:
        assert g.used <= g.capacity
    assert p.speculator == "mtp"


def test_pool_first_and_minimum():
    small = solver.PlacementRequest(qwen3_30b_a3b(), gpus=1, gpu_memory_cap=120 << 30, expert_ranks=0, attention_ranks=1)
    p = solver.solve(small)
    assert p.ok and p.kv_pool_tokens < small.pool_tokens_target and p.kv_pool_tokens >= small.pool_tokens_min
    tiny = solver.PlacementRequest(qwen3_30b_a3b(), gpus=1, gpu_memory_cap=40 << 30, expert_ranks=0, attention_ranks=1)
    q = solver.solve(tiny)
    assert not q.ok and ("over capacity" in q.reason or "KV pool" in q.reason)


def test_bf16_deepseek_does_not_fit_one_gpu():
    rep = P.plan("deepseek-v3", layout=True, fmt="bf16", gpus=1)
    assert not rep.placement.ok and not rep.ready
    assert "REJECTED" in P.render(rep)


def test_auto_prefers_disaggregation_when_experts_dominate():
    p = solver.solve(solver.PlacementRequest(deepseek_v3(), gpus=8))
    assert p.ok and p.expert_ranks > 0


def test_frozen_recheck_matches_plan():
    req = solver.PlacementRequest(qwen3_30b_a3b(), gpus=4)
    p = solver.solve(req)
    again = solver.solve_frozen(req, p.attention_ranks, p.expert_ranks, p.pipeline_stages)
    assert again.ok and again.kv_pool_tokens == p.kv_pool_tokens


def test_deployment_document_and_hash():
    rep = P.plan("qwen3-30b-a3b", layout=True, gpus=4, attention_ranks=1, expert_ranks=3)
    d = P.deployment(rep)
    assert d["world_size"] == 4 and [r["role"] for r in d["ranks"]] == ["attention", "expert", "expert", "expert"]
    assert d["ranks"][1]["experts"] == [0, 43]
    assert d["plan_hash"] == P.deployment(rep)["plan_hash"]


def test_cli_plan_json_and_snapshot(tmp_path, capsys):
    from cuteafd_b200.loader.snapshot import write_random_snapshot
    d = write_random_snapshot(tiny_moe().replace(hidden=256, expert_ffn=128), str(tmp_path / "snap"), fmt="nvfp4")
    assert main(["plan", d, "--layout", "--gpus", "2", "--json", "--pool-tokens", "4096"]) == 0
    out = json.loads(capsys.readouterr().out)
    assert out["family"] == "deepseek_v3" and out["formats"]["routed_expert"] == {"nvfp4": 24}
    assert out["placement"]["ok"]
    assert main(["plan", d, "--files", "--role", "routed_expert"]) == 0
    assert "routed_expert" in json.loads(capsys.readouterr().out)


def test_config_file_refuses_unknown_keys(tmp_path):
    f = tmp_path / "c.config"
    f.write_text("GPUS=8\n# comment\nPOOL_TOKENS = 1000\n")
    assert load_config_file(str(f), ["port=9"], {"GPUS", "POOL_TOKENS", "PORT"}) == {"GPUS": "8", "POOL_TOKENS": "1000", "PORT": "9"}
    with pytest.raises(SystemExit) as e:
        load_config_file(str(f), ["NOPE=1"], {"GPUS", "POOL_TOKENS"})
    assert e.value.code == 2


def test_auto_layout_on_one_gpu_is_the_colocated_one():
    from cuteafd_b200 import qwen3_30b_a3b
    from cuteafd_b200.planner.solver import PlacementRequest, solve
    p = solve(PlacementRequest(qwen3_30b_a3b(), gpus=1))
    assert p.ok and (p.attention_ranks, p.expert_ranks, p.engine) == (1, 0, "single")


def test_plan_names_the_engine_that_serves_it():
    from cuteafd_b200 import deepseek_v3, qwen3_30b_a3b
    from cuteafd_b200.planner.solver import PlacementRequest, engine_for, solve, solve_frozen
    q, d = qwen3_30b_a3b(), deepseek_v3()
    assert engine_for(q, 1, 7, 1)[0] == "afd" and engine_for(q, 1, 0, 1)[0] == "single"
    assert engine_for(q, 4, 0, 1)[0] == "tp" and engine_for(q, 8, 0, 1)[0] == ""        # 4 kv heads
    assert engine_for(d, 2, 6, 1)[0] == "" and engine_for(q, 1, 3, 2)[0] == ""
    assert engine_for(d, 2, 0, 1)[0] == "tp" and engine_for(d.replace(indexer_heads=64), 2, 0, 1)[0] == ""      # dense MLA heads split
    assert engine_for(q, 1, 0, 2)[0] == "pp" and engine_for(d, 1, 0, 2)[0] == ""
    best = solve(PlacementRequest(cfg=d, gpus=8))
    assert best.ok and best.engine == "afd" and best.attention_ranks == 1 and best.expert_ranks == 7
    assert any(n.startswith("served by:") for n in best.notes)
    frozen = solve_frozen(PlacementRequest(cfg=d, gpus=8), 2, 6)
    assert frozen.engine == "" and any(n.startswith("not served yet:") for n in frozen.notes)
    assert "engine" in best.to_json()


def test_graph_reserve_from_a_measured_prewarm_file(tmp_path, capsys):
    """The decode-graph arena of the layout comes from the bytes a serving run measured (base + extra) when a prewarm
    file is given, from a plain size as a user override, and from the unmeasured default otherwise."""
    import json
    from cuteafd_b200 import cli
    from cuteafd_b200.planner import plan as P
    base = P.plan("qwen3-30b-a3b", layout=True, gpus=2, attention_ranks=1, expert_ranks=1)
    g0 = base.placement.devices[0].by_category()["graphs"]
    assert g0 == 256 << 20
    pw = tmp_path / "prewarm.json"
    pw.write_text(json.dumps({"geometries": [[1, 1, 1]], "reserve_base_bytes": 900 << 20, "reserve_extra_bytes": 100 << 20}))
    nbytes, source = cli.graph_reserve_of(str(pw))
    assert nbytes == 1000 << 20 and source == "measured: prewarm.json"
    rep = P.plan("qwen3-30b-a3b", layout=True, gpus=2, attention_ranks=1, expert_ranks=1, graph_reserve_bytes=nbytes,
                 graph_reserve_source=source)
    dev = rep.placement.devices[0]
    assert dev.by_category()["graphs"] == 1000 << 20
    assert dev.free == base.placement.devices[0].free - (1000 - 256) * (1 << 20) or rep.placement.kv_pool_tokens <= base.placement.kv_pool_tokens
    assert cli.main(["plan", "qwen3-30b-a3b", "--layout", "--gpus", "2", "--attention-ranks", "1", "--expert-ranks", "1",
                     "--graph-reserve", "600MiB", "--json"]) == 0
    out = json.loads(capsys.readouterr().out)
    dev0 = out["placement"]["devices"][0]
    assert any("user override" in str(item) for item in json.dumps(dev0).split(","))
    (tmp_path / "old.json").write_text(json.dumps({"geometries": []}))
    import pytest
    with pytest.raises(SystemExit):
        cli.graph_reserve_of(str(tmp_path / "old.json"))
