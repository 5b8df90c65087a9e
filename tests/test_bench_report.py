"""Benchmark reports, cards and the published tables."""
import json
import os

import pytest

from cuteafd_b200 import cli
from cuteafd_b200.bench import report as R

LINE = {"metric": "decode_tok_s_c8", "value": 1300.0, "unit": "tok/s", "n_gpus": 8, "gpu_launches": 380,
        "config": {"model": "qwen3-30b-a3b", "parallelism": "afd: 2 replicas + ep6"},
        "clocks": {"sm_mhz": 1800, "sm_max_mhz": 1965, "reasons": ["sw_power_cap"]},
        "e2e": {"value": 1250.0}, "extra": {"prefill_tok_s": 170000.0, "ttft_s": 0.09, "decode_c1_tok_s": 190.0,
                                            "decode_c8_tok_s": 1300.0, "decode_c32_tok_s": 3300.0, "decode_c8_e2e_tok_s": 1250.0}}


def _root(tmp_path):
    (tmp_path / "benchmarks").mkdir()
    (tmp_path / "README.md").write_text(f"# x\n\n{R.RESULTS_BEGIN}\nold\n{R.RESULTS_END}\ntail\n")
    (tmp_path / "benchmarks" / "README.md").write_text(f"{R.INDEX_BEGIN}\n{R.INDEX_END}\n")
    return str(tmp_path)


def test_report_from_bench_line_and_card(tmp_path):
    root = _root(tmp_path)
    rep = R.from_bench_line(LINE, family="qwen3_moe", checkpoint="Qwen/Qwen3-30B-A3B")
    assert rep.accepted and rep.card["decode_tok_s"] == {"1": 190.0, "8": 1300.0, "32": 3300.0}
    rel = R.write_report(rep, root)
    assert rel.startswith("benchmarks/qwen3_moe/") and rel.endswith("8gpu-afd-2-replicas-ep6")
    for name in ("report.json", "card.svg", "card.md"):
        assert os.path.getsize(os.path.join(root, rel, name)) > 100
    assert "decode C32" in open(os.path.join(root, rel, "card.md")).read()
    assert "<svg" in open(os.path.join(root, rel, "card.svg")).read()
    back = R.Report.from_json(json.load(open(os.path.join(root, rel, "report.json"))))
    assert back.card == rep.card and back.accepted
    with pytest.raises(FileExistsError):
        R.write_report(rep, root)
    # a throttled run is placed but never accepted
    hot = R.from_bench_line(dict(LINE, clocks={"reasons": ["hw_thermal_slowdown"]}), family="qwen3_moe", checkpoint="hot")
    assert not hot.accepted
    with pytest.raises(ValueError):
        R.Report.from_json({"schema": "other"})


def test_report_reads_the_keys_bench_py_prints():
    line = dict(LINE, n_gpus=1, extra={"decode_tok_s_c1": 207.1, "decode_tok_s_c8": 857.0, "decode_tok_s_c32": 1745.4,
                                       "e2e_decode_tok_s_c8": 840.0, "prefill_tok_s_8k": 85714.6, "ttft_s_8k": 0.0956})
    rep = R.from_bench_line(line, family="qwen3_moe", checkpoint="c", hardware="1gpu")
    assert rep.hardware == "1gpu" and rep.card == {"prefill_tok_s": 85714.6, "ttft_s": 0.0956,
                                                   "decode_tok_s": {"1": 207.1, "8": 857.0, "32": 1745.4}}


def test_report_from_panels():
    out = {"url": "u", "ok": False, "panels": [
        {"panel": "smoke", "ok": True, "seconds": 1.0}, {"panel": "lossless", "ok": False, "error": "ids differ", "seconds": 2.0},
        {"panel": "speed", "ok": True, "prefill_tok_s": 1000.0, "prefill_ttft_s": 0.5, "c1_decode_tok_s": 50.0, "seconds": 3.0},
        {"panel": "sweep", "ok": True, "levels": {"1": {"tok_s": 55.0, "failed": 0}, "4": {"tok_s": 150.0, "failed": 0}}, "seconds": 3.0},
        {"panel": "tools", "ok": False, "seconds": 0.1}]}
    rep = R.from_panels(out, family="f", checkpoint="c", hardware="1gpu")
    assert not rep.accepted and rep.card["prefill_tok_s"] == 1000.0 and rep.card["ttft_s"] == 0.5
    assert rep.card["decode_tok_s"] == {"1": 55.0, "4": 150.0}
    assert [c["gating"] for c in rep.checks] == [True, True, False, False, False]
    out["panels"][1]["ok"] = True
    assert R.from_panels(out, family="f", checkpoint="c", hardware="1gpu").accepted      # tools is informational


def test_publish_resolves_the_matrix(tmp_path):
    root = _root(tmp_path)
    rel = R.write_report(R.from_bench_line(LINE, family="qwen3_moe", checkpoint="Qwen/Qwen3-30B-A3B"), root)
    matrix = {"schema": R.MATRIX_SCHEMA, "cells": [
        {"family": "qwen3_moe", "checkpoint": "Qwen/Qwen3-30B-A3B", "1gpu": {"status": "pending", "reason": "not measured yet"},
         "8gpu": {"status": "current", "report": rel}},
        {"family": "deepseek_v3", "checkpoint": "deepseek-ai/DeepSeek-V3", "1gpu": {"status": "na", "reason": "-"},
         "8gpu": {"status": "held", "reason": "re-measuring"}}]}
    json.dump(matrix, open(os.path.join(root, R.MATRIX_FILE), "w"))
    res = R.publish(root)
    assert res == {"reports": 1, "rows": 2, "changed": ["README.md", "benchmarks/README.md"], "current": False}
    readme = open(os.path.join(root, "README.md")).read()
    assert "C1 190.0 / C8 1,300.0 / C32 3,300.0 tok/s" in readme and "pending: not measured yet" in readme and "tail" in readme
    assert "old" not in readme and f"({rel}/card.md)" in readme
    assert "Qwen/Qwen3-30B-A3B" in open(os.path.join(root, "benchmarks", "README.md")).read()
    assert R.publish(root, check=True)["current"]
    assert cli.main(["bench", "--publish", root, "--check"]) == 0
    # a newer report does not take the cell: the matrix names the published one
    R.write_report(R.from_bench_line(dict(LINE, value=1.0), family="qwen3_moe", checkpoint="Qwen/Qwen3-30B-A3B", profile="retry"), root)
    assert R.publish(root)["changed"] == ["benchmarks/README.md"]
    # a current cell must name an accepted report of that checkpoint
    matrix["cells"][1]["8gpu"] = {"status": "current", "report": rel}
    json.dump(matrix, open(os.path.join(root, R.MATRIX_FILE), "w"))
    with pytest.raises(ValueError, match="is a report of"):
        R.publish(root)
    matrix["cells"][1]["8gpu"] = {"status": "held"}
    json.dump(matrix, open(os.path.join(root, R.MATRIX_FILE), "w"))
    with pytest.raises(ValueError, match="gives its reason"):
        R.publish(root)
    assert cli.main(["bench", "--publish", root]) == 2


def test_cli_places_a_report_from_a_saved_line(tmp_path, capsys):
    root = _root(tmp_path)
    p = tmp_path / "line.json"
    p.write_text("noise\n" + json.dumps(LINE) + "\n")
    assert cli.main(["bench", "--report-root", root, "--from-json", str(p), "--family", "qwen3_moe", "--checkpoint", "Qwen/Qwen3-30B-A3B"]) == 0
    out = json.loads(capsys.readouterr().out.strip().splitlines()[-1])
    assert out["accepted"] and os.path.exists(os.path.join(root, out["report"], "card.svg"))


def test_committed_tables_are_current():
    """The results table in the root README and the report index are what ``bench --publish .`` generates."""
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    assert R.publish(root, check=True)["current"], "run: python -m cuteafd_b200.cli bench --publish ."
