"""Launcher: deployment document -> one process per rank, supervised; configuration keys -> flags."""
import json
import os
import signal
import sys
import threading
import time

import pytest

from cuteafd_b200 import cli
from cuteafd_b200 import launch as LA


def _spec(world=3):
    import hashlib
    ranks = [{"rank": 0, "device": 0, "role": "attention", "memory": {}, "free_bytes": 0, "tp_rank": 0, "pp_stage": 0}]
    per = 16 // (world - 1)
    for r in range(1, world):
        ranks.append({"rank": r, "device": r, "role": "experts", "memory": {}, "free_bytes": 0, "experts": [(r - 1) * per, r * per]})
    body = {"model": "m", "source": "/snap", "family": "f", "layout": f"1+{world - 1}", "world_size": world, "attention_ranks": 1,
            "expert_ranks": world - 1, "pipeline_stages": 1, "rendezvous": {"master_addr": "127.0.0.1", "master_port": 29999},
            "ranks": ranks}
    body["plan_hash"] = hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()[:16]
    return json.loads(json.dumps(body))


def _child(code: str):
    return lambda spec_path, spec, entry, extra: [sys.executable, "-c", code.replace("RANK_ID", str(entry["rank"]))]


def test_validate_refuses_bad_documents():
    LA.validate(_spec())
    bad = _spec(); bad["ranks"][2]["device"] = 1
    with pytest.raises(ValueError, match="share a device"):
        LA.validate(bad)
    bad = _spec(); bad["ranks"][2]["experts"] = [9, 16]
    with pytest.raises(ValueError, match="tile"):
        LA.validate(bad)
    bad = _spec(); bad["layout"] = "edited"
    with pytest.raises(ValueError, match="plan_hash"):
        LA.validate(bad)
    bad = _spec(); bad["ranks"][0]["role"] = "experts"
    with pytest.raises(ValueError, match="rank 0"):
        LA.validate(bad)


def test_rank_environment_and_commands(tmp_path):
    L = LA.build_launch(_spec(), str(tmp_path), ["--port", "8123"])
    assert json.load(open(tmp_path / "deployment.json"))["world_size"] == 3
    assert [r.env["RANK"] for r in L.ranks] == ["0", "1", "2"] and L.ranks[2].env["LOCAL_RANK"] == "2"
    assert all(r.env["WORLD_SIZE"] == "3" and r.env["MASTER_PORT"] == "29999" for r in L.ranks)
    assert L.ranks[1].argv[-2:] == ["--port", "8123"] and "--deployment" in L.ranks[1].argv and "/snap" in L.ranks[1].argv
    assert "rank 2 [experts]" in LA.describe(L)


def test_failed_rank_takes_the_deployment_down(tmp_path):
    code = "import sys, time\nif RANK_ID == 2:\n    time.sleep(0.3); sys.exit(3)\ntime.sleep(60)"
    L = LA.build_launch(_spec(), str(tmp_path), [], argv_for=_child(code))
    L.grace_s = 1.0
    L.start()
    assert os.path.exists(L.pid_file)
    t0 = time.monotonic()
    rc = L.supervise(poll_s=0.05)
    assert rc == 3 and time.monotonic() - t0 < 20
    assert all(r.proc.poll() is not None for r in L.ranks) and not os.path.exists(L.pid_file)


def test_clean_exit_and_stop_by_pid_file(tmp_path):
    L = LA.build_launch(_spec(2), str(tmp_path / "a"), [], argv_for=_child("print('rank', RANK_ID)"))
    L.start()
    assert L.supervise(poll_s=0.05) == 0
    assert "rank 1" in open(L.ranks[1].log).read()
    # a deployment whose launcher is gone: stop signals the ranks by their recorded pids
    L2 = LA.build_launch(_spec(2), str(tmp_path / "b"), [], argv_for=_child("import time\ntime.sleep(60)"))
    L2.start()
    doc = json.load(open(L2.pid_file))
    doc["launcher"] = 0
    json.dump(doc, open(L2.pid_file, "w"))
    assert LA.stop_by_pid_file(L2.pid_file) == 0
    for r in L2.ranks:
        assert r.proc.wait(timeout=10) in (-signal.SIGINT, -signal.SIGTERM, 1, 130)


def test_launcher_stops_its_ranks_on_sigterm(tmp_path):
    L = LA.build_launch(_spec(2), str(tmp_path), [], argv_for=_child("import time\ntime.sleep(60)"))
    L.grace_s = 1.0
    L.start()
    threading.Timer(0.4, lambda: os.kill(os.getpid(), signal.SIGTERM)).start()
    assert L.supervise(poll_s=0.05) == 0
    assert all(r.proc.poll() is not None for r in L.ranks)


def test_launch_dry_run_plans_a_snapshot(tmp_path, capsys):
    from cuteafd_b200 import qwen3_30b_a3b, scaled_down
    from cuteafd_b200.loader.snapshot import write_random_snapshot
    small = scaled_down(qwen3_30b_a3b(), layers=1, vocab=512).replace(hidden=256, num_heads=2, num_kv_heads=1, num_experts=8, top_k=2,
                                                                     expert_ffn=64, name="qwen3-moe-mini")
    snap = write_random_snapshot(small, str(tmp_path / "snap"), fmt="bf16", seed=0)
    rc = cli.main(["launch", snap, "--gpus", "3", "--attention-ranks", "1", "--expert-ranks", "2", "--dry-run", "--run-dir",
                   str(tmp_path / "run"), "--port", "8111"])
    out = capsys.readouterr().out
    assert rc == 0, out
    spec = json.load(open(tmp_path / "run" / "deployment.json"))
    assert spec["world_size"] == 3 and [tuple(r["experts"]) for r in spec["ranks"][1:]] == [(0, 4), (4, 8)]
    assert out.count("cuteafd_b200.cli serve") == 3 and "--port 8111" in out
    # a geometry the CUDA kernels do not take is refused with the reason, not started
    from cuteafd_b200 import tiny_moe
    odd = write_random_snapshot(tiny_moe(), str(tmp_path / "odd"), fmt="bf16", seed=0)
    assert cli.main(["launch", odd, "--gpus", "1", "--dry-run", "--run-dir", str(tmp_path / "r0")]) == 1
    assert "fake-engine" in capsys.readouterr().err
    # an edited document is refused; the stored one starts (dry) as it is
    assert cli.main(["launch", "--deployment", str(tmp_path / "run" / "deployment.json"), "--dry-run", "--run-dir", str(tmp_path / "r2")]) == 0
    spec["world_size"] = 4
    json.dump(spec, open(tmp_path / "bad.json", "w"))
    assert cli.main(["launch", "--deployment", str(tmp_path / "bad.json"), "--dry-run", "--run-dir", str(tmp_path / "r3")]) == 2


def test_config_keys_become_flags(tmp_path):
    cfg = tmp_path / "cuteafd.config"
    cfg.write_text("MODEL=/models/x  # the checkpoint\nCONCURRENCY=3\nHTTP_QUEUE_DEPTH=7\nSPECULATOR=off\nPORT=8111\n")
    ap = cli.build_parser()
    argv = ["--config", str(cfg), "--set", "CONCURRENCY=5", "serve", "--port", "9000"]
    a = ap.parse_args(argv)
    a.file_config = cli.load_config_file(a.config, a.set, cli.CONFIG_KEYS)
    cli.apply_config(ap, a, argv)
    assert (a.snapshot, a.concurrency, a.queue_depth, a.speculator, a.port) == ("/models/x", 5, 7, "off", 9000)
    argv = ["--config", str(cfg), "launch", "--dry-run"]
    a = ap.parse_args(argv)
    a.file_config = cli.load_config_file(a.config, a.set, cli.CONFIG_KEYS)
    cli.apply_config(ap, a, argv)
    assert a.model == "/models/x" and a.concurrency == 3 and a.port == 8111
    with pytest.raises(SystemExit):
        cli.load_config_file("", ["NOPE=1"], cli.CONFIG_KEYS)
    bad = ["--set", "DECODE_LANES=5", "plan", "m"]
    a = ap.parse_args(bad)
    a.file_config = cli.load_config_file(a.config, a.set, cli.CONFIG_KEYS)
    with pytest.raises(SystemExit):
        cli.apply_config(ap, a, bad)


def test_a_rank_that_cannot_start_leaves_nothing_running(tmp_path):
    def argv_for(spec_path, spec, entry, extra):
        if entry["rank"] == 1:
            return ["/nonexistent/interpreter", "-c", "pass"]
        return [sys.executable, "-c", "import time\ntime.sleep(60)"]
    L = LA.build_launch(_spec(2), str(tmp_path), [], argv_for=argv_for)
    L.grace_s = 0.5
    with pytest.raises(OSError):
        L.start()
    assert L.ranks[0].proc.poll() is not None and L.ranks[1].proc is None


def test_a_reference_configuration_file_is_accepted(tmp_path, capsys):
    """The reference's key spellings mean the same here (units converted), "auto" leaves the default, and the keys of
    its Spark / container deployment are skipped with one notice instead of refusing the file."""
    cfg = tmp_path / "cuteafd.config"
    cfg.write_text("MODEL_ID=/models/x\nMODEL_REVISION=abc\nEXPERT_FORMAT=native\nSPECULATOR=dspark\nTP2_ATTENTION=off\nRTX_GPUS=auto\n"
                   "MAX_CONTEXT_TOKENS=auto\nCONCURRENCY=16\nHOST_CACHE_BYTES=8GiB\nHTTP_QUEUE_WAIT_MS=2500\nADDR=0.0.0.0:8123\n"
                   "SPARK_COUNT=6\nSPARK_0_HOST=ostrich\nSPARK_0_LANE_A=10.0.0.1\nCOORDINATOR_DOCKER_DEV=img\nEMBEDDING=host\n"
                   "LOOP_ABORT_RUN=256\nPREFILL_BATCH_TOKENS=2048\n")
    got = cli.load_config_file(str(cfg), [], cli.CONFIG_KEYS)
    assert got == {"MODEL": "/models/x", "SPECULATOR": "auto", "CONCURRENCY": "16", "HOST_CACHE_GIB": "8.000", "HTTP_QUEUE_WAIT": "2.5",
                   "HOST": "0.0.0.0", "PORT": "8123", "EXPERT_RANKS": "6", "EMBEDDING_PLACEMENT": "host", "LOOP_ABORT_RUN": "256",
                   "PREFILL_ROWS": "2048"}
    err = capsys.readouterr().err
    assert "skipped" in err and "SPARK_0_HOST" in err and "TP2_ATTENTION" in err
    ap = cli.build_parser()
    argv = ["--config", str(cfg), "serve"]
    a = ap.parse_args(argv)
    a.file_config = got
    cli.apply_config(ap, a, argv)
    assert (a.snapshot, a.concurrency, a.port, a.host, a.queue_wait, a.host_cache_gib, a.embedding_placement, a.loop_abort_run) == \
        ("/models/x", 16, 8123, "0.0.0.0", 2.5, 8.0, "host", 256)
    with pytest.raises(SystemExit):
        cli.load_config_file("", ["SOMETHING_ELSE=1"], cli.CONFIG_KEYS)


@pytest.mark.parametrize("name,world,engine", [("qwen3-30b-a3b-1gpu", 1, "single"), ("deepseek-v3-8gpu", 8, "afd"),
                                               ("qwen3-30b-a3b-head-split-2gpu", 2, "tp"), ("reference-style", 4, "afd")])
def test_example_configurations_plan_and_dry_run(name, world, engine, tmp_path, capsys):
    """Every shipped example is a complete launch: it parses, plans on the GPUs it names and passes the launcher's checks."""
    path = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "examples", "configs", name + ".config")
    extra = ["--gpus", "4"] if name == "reference-style" else []
    assert cli.main(["--config", path, "launch", "--dry-run", "--run-dir", str(tmp_path)] + extra) == 0
    spec = json.load(open(tmp_path / "deployment.json"))
    assert spec["world_size"] == world and spec["engine"] == engine
    out = capsys.readouterr().out
    assert out.count("cuteafd_b200.cli serve") == world


def test_serve_only_configuration_keys_reach_every_rank(tmp_path, capsys):
    """A key that is a flag of ``serve`` but not of ``launch`` becomes an argument of the ranks' serve commands; a
    --serve-arg on the launch line wins over the file; switches appear only when on."""
    from cuteafd_b200.cli import main, serve_args_from_config
    conf = tmp_path / "c.config"
    conf.write_text("MODEL=qwen3-30b-a3b\nGPUS=1\nMAX_OUTPUT_TOKENS=40\nBATCH_INVARIANT=1\nDRAFT_LENGTH=3\nDECODE_GRAPHS=off\nPORT=8123\n")
    assert main(["--config", str(conf), "launch", "--dry-run", "--run-dir", str(tmp_path / "run")]) == 0
    line = [l for l in capsys.readouterr().out.splitlines() if " serve " in l][0]
    for want in ("--max-output-tokens 40", "--batch-invariant", "--draft-length 3", "--decode-graphs off", "--port 8123"):
        assert want in line, (want, line)
    assert main(["--config", str(conf), "launch", "--dry-run", "--run-dir", str(tmp_path / "run"), "--serve-arg=--draft-length", "--serve-arg=5"]) == 0
    line = [l for l in capsys.readouterr().out.splitlines() if " serve " in l][0]
    assert "--draft-length 5" in line and "--draft-length 3" not in line
    assert serve_args_from_config({"BATCH_INVARIANT": "0", "MODEL": "x", "GPUS": "2"}, []) == []
    with pytest.raises(SystemExit):
        serve_args_from_config({"DECODE_GRAPHS": "sometimes"}, [])
