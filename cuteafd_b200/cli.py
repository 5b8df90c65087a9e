"""``cuteafd`` command line: plan | serve | expertd | golden | bench | fabric | doctor | gateway | usage | mc | prewarm.

    python -m cuteafd_b200.cli plan deepseek-v3 --layout --gpus 8
    python -m cuteafd_b200.cli plan /path/to/snapshot --layout --deployment
    python -m cuteafd_b200.cli serve --snapshot /path/to/snapshot --port 8000
    python -m cuteafd_b200.cli bench --gpus 1

Counterpart: rust/crates/cuteafd-daemon/src/cli.rs:133-295 (Commands), main.rs:363-641 (dispatch),
commands/plan.rs.  Options may also come from ``KEY=VALUE`` config files (``--config``) with
``--set KEY=VALUE`` overrides; unknown keys are refused, as the reference launcher does
(docs/options.md:210-232).
"""
from __future__ import annotations

import argparse
import json
import os
import sys


def _size(s: str) -> int:
    s = s.strip().lower()
    for suf, mul in (("gib", 1 << 30), ("gb", 10 ** 9), ("mib", 1 << 20), ("mb", 10 ** 6), ("g", 1 << 30), ("m", 1 << 20)):
        if s.endswith(suf):
            return int(float(s[: -len(suf)]) * mul)
    return int(s)


def _size_bytes(s: str) -> int:
    """Sizes as the reference writes them: decimal or binary units, fractions allowed (22.5GB, 90GiB, 512MiB, 1048576B)."""
    t = s.strip().lower()
    if t.endswith("b") and not t.endswith(("gb", "mb", "kb", "ib")):
        t = t[:-1]
    if t.endswith("kib"):
        return int(float(t[:-3]) * 1024)
    if t.endswith("kb"):
        return int(float(t[:-2]) * 1000)
    return _size(t)


def _gib(v: str) -> str:
    return f"{_size(v) / (1 << 30):.3f}"


# Spellings of the reference's configuration file (cuteafd.config: run.sh --config / --set) -> this framework's keys, with
# a converter for the value where the unit differs.  A reference configuration is accepted as it is: "auto" leaves the
# default in place, and keys that describe what this framework does not have (Spark hosts and rails, container images,
# SSH, the coordinator's GPU pick, TP2 switches of the RTX pair) are skipped with one notice.
REFERENCE_KEYS = {
    "MODEL_ID": ("MODEL", None), "EMBEDDING": ("EMBEDDING_PLACEMENT", None), "RTX_GPUS": ("ATTENTION_RANKS", None),
    "SPARK_COUNT": ("EXPERT_RANKS", None), "KV_TARGET_TOKENS": ("POOL_TOKENS", None), "PREFILL_BATCH_TOKENS": ("PREFILL_ROWS", None),
    "HTTP_QUEUE_WAIT_MS": ("HTTP_QUEUE_WAIT", lambda v: str(float(v) / 1000.0)), "HOST_CACHE_BYTES": ("HOST_CACHE_GIB", _gib),
    "KV_POOL_TOKENS": ("POOL_TOKENS", None), "SPECULATOR_MODEL_ID": ("DRAFT_SNAPSHOT", None), "GRAPH_PREWARM": ("PREWARM", None),
    "GPU_GRAPH_RESERVE": ("GRAPH_RESERVE", None),
}
# Keys the reference documents (docs/options.md of its tree) that have no counterpart here: family-specific kernel
# switches, its profiler wrappers, Spark / RDMA / container settings, graph-donor and padding policies.  They are skipped
# with the notice, so a configuration written for it still starts.
REFERENCE_ONLY = frozenset("""ATTENTION_PLACEMENT ATTENTION_PLAN_ROWS ATTENTION_PRECISION AUDIO_FEATURES_DIR AUDIO CHAT_TEMPLATE_FROM
CONSOLE_ASSETS CONSOLE_TEXT CUDA_MODULE_LOADING DRAFT_CONTEXT_SLOTS DRAFT_CONTEXT_WINDOW DRAFT_KV_CACHE DRAFT_POLICY
DRAFT_SEQUENCES ENABLE_BENCH ENGRAM_WARM EXLR8_MANIFEST EXLR8_PREFILL_ACTIVATIONS EXPERT_BACKEND EXPERT_INPUT
EXPERT_PARTIAL_BF16_MAX_ROWS EXPERT_USAGE FAMILY_RESERVE FP8_PREFILL FP8_SCALES GATEWAY GPU_GRAPH_RESERVE_EXTRA_CAP
GPU_GRAPH_RESERVE_EXTRA GPU_RESERVE GRAPH_DISABLE_LOW_MEM GRAPH_DONOR_ALWAYS GRAPH_DONOR_COLD_LAG GRAPH_NODE_PADDING GRAPH_TRACE
HOST_ISA HOST_WAIT IDLE_PARK_SECONDS KV_CACHE L2_PREFETCH MAPPED_SCALE_PRELOAD_GIB MEDIA_CACHE_BYTES MEDIA_FEATURES_DIR
MEMORY_PADDING PREFILL_PACKING PREFILL_SPAN_ROWS PREFILL_WAVES PREFIX_CACHE_MARK_MIB PREFIX_PARTIAL PREFIX_POINT_BOUNDARIES
PROBE_DUMP_ROOT RDMA_BOND_BALANCE SPECULATOR_DEPTH SPECULATOR_FP8 SPECULATOR_MODEL_REVISION SWA_KV_CACHE TARGET_HEAD THERMAL
USAGE VISION_REPLICAS VISION V41_FP8_HEAD QWEN_FP8_DECODE QWEN_FP8_HEAD""".split())
REFERENCE_ONLY_PREFIXES = ("GLM5_FLASH_", "MIMO_", "PROFILE_N", "PROFILE_SPARK", "PROFILE_EXPERT_", "WIP_")
REFERENCE_SKIPPED = ("SPARK_", "COORDINATOR_", "SPARKINFER_", "TP2_", "CUTEAFD_", "MODEL_VARIANT", "MODEL_REVISION", "EXPERT_PORT",
                     "INSTANCE", "KV_MIN_TOKENS", "KV_MAX_TOKENS",
                     "KV_RESERVE_DRAIN_BUFFER",
                     "RTX_EXPERT_LAYERS", "FULL_PREFILL_LOGITS")
REFERENCE_SPECULATORS = {"dspark": "auto", "dflash2": "auto"}      # trained block drafters of the reference's checkpoints


def _speculator(v: str) -> str:
    """``--speculator`` of plan / launch: the reference's trained block drafters (dspark, dflash2) plan as ``auto``."""
    return REFERENCE_SPECULATORS.get(v.lower(), v)


def reference_key(k: str, v: str, skipped: list[str]) -> list[tuple[str, str]]:
    """One line of a reference configuration -> the (key, value) pairs it means here ([] = nothing to set)."""
    if k == "ADDR":                                           # host:port of the HTTP listener
        host, _, port = v.rpartition(":")
        return ([("HOST", host)] if host else []) + ([("PORT", port)] if port else [])
    if k == "API_KEY_FILE":                                   # the bearer key kept out of the configuration file
        with open(os.path.expanduser(v)) as f:
            return [("API_KEY", f.read().strip())]
    if k in REFERENCE_ONLY or k.startswith(REFERENCE_ONLY_PREFIXES):
        skipped.append(k)
        return []
    if k == "SPARK_COUNT" or not (k.endswith("_DOCKER_DEV") or k.endswith("_DOCKER_INFERENCE") or k.startswith(REFERENCE_SKIPPED)):
        name, conv = REFERENCE_KEYS.get(k, (k, None))
        if v.lower() == "auto" and name not in ("SPECULATOR",):
            return []                                         # the planner / the flag's default decides
        if name == "SPECULATOR":
            v = REFERENCE_SPECULATORS.get(v.lower(), v)
        if name == "EXPERT_FORMAT" and v.lower() == "native":
            return []                                         # "as stored" is what the loader does without an override
        return [(name, conv(v) if conv else v)]
    skipped.append(k)
    return []


def load_config_file(path: str, overrides: list[str], known: set[str]) -> dict[str, str]:
    """KEY=VALUE file + ``--set`` overrides; the reference's spellings are translated (``REFERENCE_KEYS``), its
    hardware-specific keys skipped with a notice; any other unknown key exits with status 2."""
    out: dict[str, str] = {}
    skipped: list[str] = []
    lines = []
    if path:
        with open(path) as f:
            lines = f.read().splitlines()
    for raw in list(lines) + list(overrides):
        line = raw.split("#", 1)[0].strip()
        if not line:
            continue
        if "=" not in line:
            print(f"config: malformed line {raw!r}", file=sys.stderr)
            raise SystemExit(2)
        k, v = line.split("=", 1)
        for k, v in reference_key(k.strip().upper(), v.strip(), skipped):
            if k not in known:
                print(f"config: unknown key {k}", file=sys.stderr)
                raise SystemExit(2)
            out[k] = v
    if skipped:
        print(f"config: {len(skipped)} key(s) of the reference's deployment that have no counterpart here were skipped: "
              + ", ".join(sorted(set(skipped))[:8]) + (" ..." if len(set(skipped)) > 8 else ""), file=sys.stderr)
    return out


CONFIG_KEYS = {"MODEL", "EMBEDDING_PLACEMENT", "GPUS", "ATTENTION_RANKS", "EXPERT_RANKS", "POOL_TOKENS", "GPU_MEMORY_CAP", "MAX_CONTEXT_TOKENS",
               "CONCURRENCY", "SPECULATOR", "DECODE_LANES", "PORT", "HOST", "API_KEY", "DECODE_SHARE", "PREFILL_ROWS",
               "HTTP_QUEUE_DEPTH", "HTTP_QUEUE_WAIT", "PROFILE", "SPECULATION_TRACE", "KV_FORMAT", "EXPERT_FORMAT",
               "HOST_CACHE_GIB", "LOOP_ABORT_RUN", "LOOP_ABORT_COPIES", "LOOP_FAST_SPAN", "LOOP_FAST_COPIES", "BATCH_INVARIANT",
               "MAX_OUTPUT_TOKENS", "KV_DECODE_RESERVE_CHUNK", "PREFIX_CACHE_ENTRIES", "KV_POOL_SIZE",
               "KV_EARLY_TERMINATION_MIN_OUTPUT_TOKENS", "DRAFT_LENGTH", "DRAFT_SNAPSHOT", "PREWARM", "GRAPH_RESERVE", "PROFILE_DIR",
               "SERVED_MODEL_ID", "DECODE_GRAPHS", "CORE_VIEW"}


def graph_reserve_of(value: str) -> tuple[int, str]:
    """``--graph-reserve``: a prewarm file a serving run saved (its measured base + extra bytes) or a plain size."""
    if os.path.exists(value):
        with open(value) as f:
            doc = json.load(f)
        if "reserve_base_bytes" not in doc:
            print(f"plan: {value} carries no measured graph bytes (written by an older run?)", file=sys.stderr)
            raise SystemExit(2)
        return int(doc["reserve_base_bytes"]) + int(doc.get("reserve_extra_bytes", 0)), f"measured: {os.path.basename(value)}"
    return _size(value), "user override"


CORE_VIEWS = ("original", "k8-compact", "k6-compact", "fp8-compact")


def _core_view(a: argparse.Namespace) -> None:
    """``--core-view``: which dense-core variant of a multi-core repository this process opens (read by the loader)."""
    if getattr(a, "core_view", None):
        os.environ["CUTEAFD_CORE_VIEW"] = a.core_view


def cmd_plan(a: argparse.Namespace) -> int:
    from .planner import plan as P
    _core_view(a)
    if a.file_layout:
        # host layout: every host's shares (attention, experts:lo:hi, a role name) as one slice per host
        from .loader import slice as SL
        try:
            hosts = SL.read_layout(a.file_layout)
            if a.host:
                if a.host not in hosts:
                    raise ValueError(f"host {a.host!r} is not in the layout ({', '.join(sorted(hosts))})")
                hosts = {a.host: hosts[a.host]}
            out = {}
            for host, sels in hosts.items():
                if a.fetch and not a.dry_run:
                    dst = a.fetch if a.host else os.path.join(a.fetch, host)
                    out[host] = SL.slice_snapshot(a.model, dst, selectors=sels, force=a.force)
                else:
                    out[host] = SL.inventory(a.model, sels)
        except (ValueError, OSError) as e:
            print(f"plan: {e}", file=sys.stderr)
            return 2
        print(json.dumps(out, indent=1))
        return 0
    if a.fetch:
        from .loader import slice as SL
        er = tuple(int(v) for v in a.expert_range.split(":")) if a.expert_range else None
        sel = dict(roles={r for r in a.role.split(",") if r} or None, exclude={r for r in a.exclude_role.split(",") if r} or None,
                   expert_range=er)
        info = SL.inventory(a.model, [sel]) if a.dry_run else SL.slice_snapshot(a.model, a.fetch, force=a.force, **sel)
        print(json.dumps(info, indent=1))
        return 0
    kw = dict(gpus=a.gpus, attention_ranks=a.attention_ranks, expert_ranks=a.expert_ranks, pool_tokens_target=a.pool_tokens,
              kv_pool_bytes=_size_bytes(a.kv_pool_size) if getattr(a, "kv_pool_size", "") else None,
              gpu_memory_cap=_size(a.gpu_memory_cap) if a.gpu_memory_cap else None, max_context_tokens=a.max_context_tokens,
              concurrency=a.concurrency, speculator=a.speculator, decode_lanes=a.decode_lanes,
              pipeline_stages=a.pipeline_stages, expert_format=a.expert_format, kv_format=a.kv_format)
    if a.graph_reserve:
        kw["graph_reserve_bytes"], kw["graph_reserve_source"] = graph_reserve_of(a.graph_reserve)
    rep = P.plan(a.model, layout=a.layout or a.deployment, fmt=a.format, **kw)
    if a.deployment:
        if not (rep.placement and rep.placement.ok):
            print(P.render(rep), file=sys.stderr)
            return 1
        print(json.dumps(P.deployment(rep), indent=1))
    elif a.files:
        files = rep.role_files if not a.role else {a.role: rep.role_files.get(a.role, [])}
        print(json.dumps(files, indent=1))
    elif a.json:
        print(json.dumps(P.to_json(rep), indent=1, default=str))
    else:
        print(P.render(rep))
    return 0 if (rep.ready or not a.require_ready) else 1


def cmd_serve(a: argparse.Namespace) -> int:
    from .serve.server import run_server
    _core_view(a)
    if getattr(a, "batch_invariant", False):
        os.environ["CAFD_BATCH_INVARIANT"] = "1"         # read by the engines when they are built
    return run_server(a)


def cmd_launch(a: argparse.Namespace) -> int:
    """Plan, write the deployment document, start one ``serve`` per rank and supervise them."""
    from . import launch as LA
    from .planner import plan as P
    _core_view(a)
    if a.deployment:
        with open(a.deployment) as f:
            spec = json.load(f)
    else:
        if not a.model:
            print("launch: name a MODEL (argument or configuration key) or pass --deployment FILE", file=sys.stderr)
            return 2
        rep = P.plan(a.model, layout=True, gpus=a.gpus, attention_ranks=a.attention_ranks, expert_ranks=a.expert_ranks,
                     pool_tokens_target=a.pool_tokens, gpu_memory_cap=_size(a.gpu_memory_cap) if a.gpu_memory_cap else None,
                     kv_pool_bytes=_size_bytes(a.kv_pool_size) if getattr(a, "kv_pool_size", "") else None,
                     max_context_tokens=a.max_context_tokens, concurrency=a.concurrency, speculator=a.speculator,
                     decode_lanes=a.decode_lanes)
        if not (rep.placement and rep.placement.ok and rep.ready):
            print(P.render(rep), file=sys.stderr)
            return 1
        from .planner.solver import HTTP_ENGINES
        if rep.placement.engine not in HTTP_ENGINES:
            print(P.render(rep), file=sys.stderr)
            print(f"launch: the HTTP server drives one attention rank (layouts {' / '.join(HTTP_ENGINES)}); this plan is "
                  f"{rep.placement.engine or 'not served by an engine'} - give --attention-ranks 1", file=sys.stderr)
            return 1
        spec = P.deployment(rep, a.master_addr, a.master_port)
    serve_args = ["--host", a.host, "--port", str(a.port)]
    if a.api_key:
        serve_args += ["--api-key", a.api_key]
    for flag, val in (("--max-context-tokens", a.max_context_tokens), ("--concurrency", a.concurrency)):
        if val is not None:
            serve_args += [flag, str(val)]
    if a.speculator:
        serve_args += ["--speculator", a.speculator]
    if getattr(a, "core_view", None):
        serve_args += ["--core-view", a.core_view]
    serve_args += serve_args_from_config(getattr(a, "file_config", {}), serve_args + list(a.serve_arg))
    serve_args += list(a.serve_arg)
    try:
        L = LA.build_launch(spec, a.run_dir, serve_args)
    except ValueError as e:
        print(f"launch: {e}", file=sys.stderr)
        return 2
    print(LA.describe(L), flush=True)
    if a.dry_run:
        return 0
    L.start()
    print(f"[launch] {len(L.ranks)} ranks started; logs and pid file under {a.run_dir}", flush=True)
    return L.supervise()


def cmd_stop(a: argparse.Namespace) -> int:
    from . import launch as LA
    path = os.path.join(a.run_dir, "launch.json")
    if not os.path.exists(path):
        print(f"stop: no deployment recorded under {a.run_dir}", file=sys.stderr)
        return 1
    return LA.stop_by_pid_file(path)


def cmd_expertd(a: argparse.Namespace) -> int:
    from .serve.expertd import run_expertd
    return run_expertd(a)


def cmd_golden(a: argparse.Namespace) -> int:
    if getattr(a, "layer_major", ""):
        import torch

        from .loader.load import open_snapshot
        from .ref import layer_major as LM
        if not a.snapshot:
            print("golden --layer-major reads a checkpoint: give --snapshot", file=sys.stderr)
            return 2
        vocab = open_snapshot(a.snapshot).cfg.vocab_size
        toks = torch.randint(0, vocab, (a.windows, a.tokens), generator=torch.Generator().manual_seed(1))
        print(json.dumps(LM.run(a.snapshot, toks, a.layer_major, log=lambda m: print(f"[golden] {m}", file=sys.stderr, flush=True))))
        return 0
    from .bench.golden import run_golden
    return run_golden(a)


def _build_id() -> str:
    """Short id of the source tree a report was produced by (the git commit when there is one)."""
    import subprocess
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    try:
        return subprocess.run(["git", "-C", root, "rev-parse", "--short", "HEAD"], capture_output=True, text=True, timeout=5).stdout.strip()
    except (OSError, subprocess.SubprocessError):
        return ""


def cmd_bench(a: argparse.Namespace) -> int:
    import subprocess
    if a.publish:                              # rebuild the generated tables from the reports on disk
        from .bench import report as R
        try:
            res = R.publish(a.publish, check=a.check)
        except (ValueError, OSError) as e:
            print(f"bench publish: {e}", file=sys.stderr)
            return 2
        print(json.dumps(res))
        return 0 if (res["current"] or not a.check) else 1
    if a.report_root and a.from_json:          # a saved bench.py line becomes a placed report
        from .bench import report as R
        with open(a.from_json) as f:
            line = json.loads([ln for ln in f.read().splitlines() if ln.strip().startswith("{")][-1])
        model = (line.get("config") or {}).get("model", "model")
        rep = R.from_bench_line(line, family=a.family or model, checkpoint=a.checkpoint or model, profile=a.profile_name, build=_build_id(),
                                hardware=a.hardware)
        print(json.dumps({"report": R.write_report(rep, a.report_root), "accepted": rep.accepted}))
        return 0
    if a.url:                                  # panels against a live server, over its HTTP API
        from .bench import panels
        names = []
        for p in a.panels.split(","):                # "quick" stands for the first five, alone or inside a list
            names += list(panels.QUICK) if p == "quick" else ([p] if p else [])
        opts = {"max_tokens": a.max_tokens, "levels": [int(v) for v in a.levels.split(",") if v], "seconds": a.seconds,
                "concurrency": a.concurrency, "windows": a.windows, "kl_bar": a.kl_bar, "top1_bar": a.top1_bar,
                "fidelity_windows": a.fidelity_windows, "lengths": [int(v) for v in a.lengths.split(",") if v], "vocab": a.vocab,
                "sessions": a.sessions, "turns": a.turns}
        out = panels.run(a.url, names, a.bench_api_key, opts)
        res = {"ok": out["ok"], "panels": len(out["panels"])}
        if a.report_root:
            from .bench import report as R
            rep = R.from_panels(out, family=a.family or "model", checkpoint=a.checkpoint or a.family or "model",
                                hardware=a.hardware or "1gpu", profile=a.profile_name, build=_build_id())
            res.update(report=R.write_report(rep, a.report_root), accepted=rep.accepted)
        print(json.dumps(res))
        return 0 if out["ok"] else 1
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    cmd = [sys.executable, os.path.join(root, "bench.py"), "--gpus", str(a.gpus), "--steps", str(a.steps), "--warmup", str(a.warmup)]
    if a.gpus > 1:
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={a.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", str(a.port)] + cmd[1:]
    return subprocess.call(cmd)


def cmd_fabric(a: argparse.Namespace) -> int:
    from .parallel.fabric import fabric_report
    rep = fabric_report(p2p=a.p2p)
    print(json.dumps(rep, indent=1) if a.json else "\n".join(f"{k}: {v}" for k, v in rep.items()))
    return 0


def cmd_doctor(a: argparse.Namespace) -> int:
    from .utils.doctor import doctor
    ok, lines = doctor()
    print("\n".join(lines))
    return 0 if ok else 1


def cmd_mc(a: argparse.Namespace) -> int:
    from .loader import mc, snapshot
    try:
        d = snapshot.resolve(a.directory)
        if a.action == "validate":
            print(json.dumps(mc.validate(d), indent=1))
            return 0
        m = mc.discover(d)
        if m is None:
            print(f"{d}: a plain checkpoint (no {mc.DISCOVERY}); its only core view is original")
            return 0
        for name, v in m.variants.items():
            print(f"{name:<12} {v.core_bits:>2} bits  {len(v.core_tensors):>5} core tensors  index {v.index}  fingerprint {v.fingerprint[:16]}")
        print(f"{'fp8-compact':<12}  8 bits  derived from original at load ({mc.FP8_RECIPE})")
        return 0
    except (mc.McError, OSError) as e:
        print(f"mc: {e}", file=sys.stderr)
        return 1


def cmd_prewarm(a: argparse.Namespace) -> int:
    from .utils.trace import prewarm_from_trace
    try:
        doc = prewarm_from_trace(a.trace, a.top)
    except OSError as e:
        print(f"prewarm: {e}", file=sys.stderr)
        return 1
    text = json.dumps(doc, indent=1)
    if a.out:
        with open(a.out, "w") as f:
            f.write(text + "\n")
        print(f"{len(doc['geometries'])} geometries from {doc['rounds']} rounds -> {a.out}")
    else:
        print(text)
    return 0


def cmd_gateway(a: argparse.Namespace) -> int:
    from .serve.gateway import run_gateway
    return run_gateway(a)


def cmd_quantize(a: argparse.Namespace) -> int:
    from .quant.quantize import QUANT_ROLES, Recipe, merge, quantize_snapshot
    roles = {r: getattr(a, r) for r in QUANT_ROLES if getattr(a, r) != "keep"}
    recipe = Recipe(roles, seed=a.seed)
    if not a.merge_only:
        quantize_snapshot(a.src, a.dst, recipe, a.rank, a.world, a.device, hessians=a.hessians or None)
    if a.merge_only or a.world == 1:
        m = merge(a.src, a.dst, recipe, a.world)
        print(json.dumps(m["summary"]))
    return 0


def cmd_calibrate(a: argparse.Namespace) -> int:
    from .loader.load import load_params
    from .quant import calibrate
    from .serve.tokenizer import load_tokenizer
    cfg, params = load_params(a.src, dtype=torch_dtype(a.dtype))
    tok = load_tokenizer(a.src, cfg.vocab_size) if a.tokens else None
    col = calibrate.collect(cfg, params, calibrate.token_batches(a.tokens or None, tok, cfg.vocab_size, a.rows, a.seq, a.seed))
    files = calibrate.save(col, a.dst)
    print(json.dumps({"operands": len(col.h), "rows_min": min(col.rows.values()), "rows_max": max(col.rows.values()),
                      "files": files}))
    return 0


def torch_dtype(name: str):
    import torch
    return {"f32": torch.float32, "bf16": torch.bfloat16}[name]


def cmd_encoderd(a: argparse.Namespace) -> int:
    """Media encoder service: holds the vision / audio towers of a snapshot and serves embedding rows over TCP."""
    import time

    import torch

    from .loader.snapshot import read_config
    from .media.loader import load_towers
    from .media.remote import EncoderServer
    cfg, _ = read_config(a.snapshot) if a.snapshot else (None, None)
    hidden = cfg.hidden if cfg else a.hidden
    dev = a.device if (a.device == "cpu" or torch.cuda.is_available()) else "cpu"
    vision, audio = load_towers(a.snapshot, hidden, dev) if a.snapshot else (None, None)
    if a.random:
        from .media import AudioTower, AudioTowerConfig, VisionTower, VisionTowerConfig
        small = dict(width=256, depth=2, heads=4, mlp=512, out_hidden=hidden)
        vision = vision or VisionTower(VisionTowerConfig(**small), VisionTower.random_weights(VisionTowerConfig(**small)), dev)
        audio = audio or AudioTower(AudioTowerConfig(**small), AudioTower.random_weights(AudioTowerConfig(**small)), dev)
    if vision is None and audio is None:
        raise SystemExit("the snapshot bundles no vision or audio tower (use --random for random-init towers)")
    srv = EncoderServer(vision, audio, a.host, a.port).start()
    print(f"media encoder ({'vision' if vision else ''}{'+' if vision and audio else ''}{'audio' if audio else ''}) on {a.host}:{srv.port}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()
    return 0


def cmd_fidelity(a: argparse.Namespace) -> int:
    from .bench.fidelity import run_cli
    return run_cli(a)


def cmd_usage(a: argparse.Namespace) -> int:
    from .serve.usage import usage_report
    print(json.dumps(usage_report(a.db, a.hours), indent=1))
    return 0


# Help for flags declared without one; keyed by destination, or by (subcommand, destination) where the meaning differs.
_HELP = {
    "set": "override one configuration key (repeatable); wins over --config",
    "model": "snapshot directory, Hugging Face cache name, or a preset name",
    "layout": "print the per-GPU memory layout (weights by role, KV pool, workspaces, graphs)",
    ("plan", "json"): "print the plan as JSON", ("fabric", "json"): "print the report as JSON",
    ("plan", "deployment"): "print the typed launch description (one entry per rank) as JSON",
    ("expertd", "deployment"): "launch description written by plan --deployment (expert ranges, peers)",
    "files": "list the checkpoint files (and byte ranges) each role needs",
    "role": "restrict --files to one role (attention, experts, head, ...)",
    "require_ready": "exit 1 when a tensor has no kernel that serves its format",
    ("plan", "gpus"): "GPUs of the box to plan for", ("bench", "gpus"): "GPUs to run the benchmark on",
    "attention_ranks": "GPUs that run attention and the dense backbone (default: solver's choice)",
    "expert_ranks": "GPUs that hold routed experts (default: solver's choice)",
    "pipeline_stages": "split the layers into this many pipeline stages",
    "pool_tokens": "KV pool size in tokens (default: what memory allows, at least 256K)",
    "gpu_memory_cap": "usable memory per GPU, e.g. 160GiB (default: all of it less a safety margin)",
    ("plan", "max_context_tokens"): "longest context a request may reach (sizes workspaces)",
    ("serve", "max_context_tokens"): "longest context a request may reach (sizes the KV pool and workspaces)",
    ("plan", "concurrency"): "requests decoded together (sizes graphs and workspaces)",
    ("serve", "concurrency"): "requests decoded together; more wait in the admission queue",
    ("plan", "speculator"): "speculative decoding to plan memory for",
    ("serve", "speculator"): "auto (MTP depth of the checkpoint, else history n-gram), history, ngram, mtp, draft-model (a small checkpoint drafts token by token), block-draft (it drafts the block in one pass), off",
    "decode_lanes": "independent decode batches served alternately",
    "format": "override the detected storage format of dense weights",
    "expert_format": "override the detected storage format of routed experts",
    ("plan", "kv_format"): "KV record format to plan for (bf16, fp8_ds_mla)",
    ("serve", "kv_format"): "KV record format: auto picks the 656-byte FP8 latent record for sparse-attention checkpoints",
    ("serve", "snapshot"): "checkpoint to serve (default: random-init weights of --preset)",
    ("expertd", "snapshot"): "checkpoint to read this rank's experts from",
    ("golden", "snapshot"): "checkpoint to compare (default: random-init weights of --preset)",
    ("serve", "preset"): "architecture preset when no snapshot is given", ("golden", "preset"): "architecture preset when no snapshot is given",
    ("serve", "host"): "address to listen on", ("gateway", "host"): "address to listen on",
    ("serve", "port"): "port to listen on", ("gateway", "port"): "port to listen on",
    ("bench", "port"): "rendezvous port for multi-GPU runs",
    "api_key": "require this bearer token (default: $CUTEAFD_API_KEY; empty = no authentication)",
    "layers": "serve only the first N layers of a preset (smoke runs)",
    "queue_depth": "requests that may wait for admission; further ones get HTTP 429",
    "queue_wait": "seconds a request may wait for admission before HTTP 429",
    "usage_db": "sqlite file for request accounting (empty = off)",
    ("expertd", "rank"): "this worker's rank in the job", ("expertd", "world"): "ranks in the job",
    ("quantize", "rank"): "this worker's index", ("quantize", "world"): "workers that share the operands",
    "master_addr": "rendezvous address", "master_port": "rendezvous port",
    ("golden", "tokens"): "tokens in the comparison prompt", "out": "write the per-layer report to this JSON file",
    "steps": "timed steps", "warmup": "untimed warm-up steps",
    "p2p": "also time a 256 MiB peer copy between GPU 0 and GPU 1",
    "upstream": "OpenAI-compatible server the gateway forwards to",
    "model_map": "comma-separated client=upstream model name pairs",
    ("quantize", "src"): "source snapshot", ("quantize", "dst"): "output directory",
    ("calibrate", "src"): "snapshot to run", ("calibrate", "dst"): "output directory for the Hessian shards",
    "device": "device the encoders run on (cpu, cuda:0, ...)",
    ("quantize", "seed"): "seed of the EXL3 sign flips", ("calibrate", "seed"): "seed of the random-id fallback",
    "rows": "calibration tokens in total", "seq": "tokens per calibration sequence",
    "dtype": "precision the oracle decoder runs in",
    "db": "sqlite file written by serve --usage-db", "hours": "window of the report",
}


def _fill_help(ap: argparse.ArgumentParser) -> None:
    subs = next(a for a in ap._actions if isinstance(a, argparse._SubParsersAction))
    for name, sp in [("", ap)] + list(subs.choices.items()):
        for a in sp._actions:
            if a.help is None:
                a.help = _HELP.get((name, a.dest), _HELP.get(a.dest))


def build_parser() -> argparse.ArgumentParser:
    ap = _build_parser()
    _fill_help(ap)
    return ap


def _build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="cuteafd", description="B200-native attention/FFN-disaggregated MoE serving")
    ap.add_argument("--config", default="", help="KEY=VALUE file")
    ap.add_argument("--set", action="append", default=[], metavar="KEY=VALUE")
    sub = ap.add_subparsers(dest="cmd", required=True)

    p = sub.add_parser("plan", help="describe a checkpoint and lay it out on the GPUs")
    p.add_argument("model")
    p.add_argument("--layout", action="store_true"); p.add_argument("--json", action="store_true")
    p.add_argument("--deployment", action="store_true"); p.add_argument("--files", action="store_true")
    p.add_argument("--role", default=""); p.add_argument("--require-ready", action="store_true")
    p.add_argument("--fetch", default="", help="copy the slice named by --role / --exclude-role / --expert-range into this directory, byte for byte")
    p.add_argument("--exclude-role", default="", help="with --fetch: comma-separated roles to leave out")
    p.add_argument("--expert-range", default="", help="with --fetch: first:end of the routed experts to keep")
    p.add_argument("--gpus", type=int, default=8); p.add_argument("--attention-ranks", type=int, default=None)
    p.add_argument("--expert-ranks", type=int, default=None); p.add_argument("--pipeline-stages", type=int, default=1)
    p.add_argument("--pool-tokens", type=int, default=None); p.add_argument("--gpu-memory-cap", default="")
    p.add_argument("--kv-pool-size", default="", help="KV pool target as a size per attention GPU (22.5GB, 90GiB) instead of --pool-tokens")
    p.add_argument("--max-context-tokens", type=int, default=None); p.add_argument("--concurrency", type=int, default=None)
    p.add_argument("--core-view", default=None, choices=CORE_VIEWS, help="dense-core variant of a multi-core checkpoint (cuteafd-mc.json): the source core, a stored 8- / 6-bit trellis core, or the source core encoded to E4M3 block-128 at load")
    p.add_argument("--file-layout", default="", help='JSON host-to-shares map, e.g. {"boxA": ["attention", "experts:0:64"]}: lists '
                                                     "(or with --fetch copies) what each host has to hold")
    p.add_argument("--host", default="", help="with --file-layout: this host only (--fetch then writes straight into its directory)")
    p.add_argument("--dry-run", action="store_true", help="with --fetch: print tensors, bytes and source files, copy nothing")
    p.add_argument("--force", action="store_true", help="with --fetch: rewrite a destination that already holds this selection")
    p.add_argument("--speculator", default=None, type=_speculator, choices=["auto", "off", "mtp"]); p.add_argument("--decode-lanes", type=int, default=None, choices=[1, 2])
    p.add_argument("--format", default=None); p.add_argument("--expert-format", default=None); p.add_argument("--kv-format", default=None)
    p.add_argument("--graph-reserve", default="", help="decode-graph arena per attention GPU: a prewarm file saved by a serving run "
                                                      "(its measured bytes) or a size such as 600MiB (default: 256 MiB per lane, unmeasured)")
    p.set_defaults(fn=cmd_plan)

    s = sub.add_parser("serve", help="HTTP serving (OpenAI / Anthropic compatible)")
    s.add_argument("--snapshot", default=""); s.add_argument("--preset", default="")
    s.add_argument("--deployment", default="", help="deployment document (plan --deployment / launch): how many attention ranks the group has, pool and row budgets")
    s.add_argument("--host", default="127.0.0.1"); s.add_argument("--port", type=int, default=8000)
    s.add_argument("--api-key", default=os.environ.get("CUTEAFD_API_KEY", ""))
    s.add_argument("--max-context-tokens", type=int, default=16384); s.add_argument("--concurrency", type=int, default=8)
    s.add_argument("--speculator", default="auto"); s.add_argument("--layers", type=int, default=0)
    s.add_argument("--core-view", default=None, choices=CORE_VIEWS, help="dense-core variant of a multi-core checkpoint (cuteafd-mc.json): the source core, a stored 8- / 6-bit trellis core, or the source core encoded to E4M3 block-128 at load")
    s.add_argument("--expert-workers", default="", help="host:port:first:end,... routed experts served by expertd --tcp-port workers "
                                                        "(host reference backend; the ranges must partition the experts)")
    s.add_argument("--served-model-id", default="", help="the model id /v1/models and replies carry (default: the checkpoint's name)")
    s.add_argument("--decode-graphs", default="on", choices=["on", "off"], help="off: every decode step runs eagerly (no CUDA graph bank)")
    s.add_argument("--draft-length", type=int, default=4, help="tokens the history / draft-model drafters propose per round (1..16)")
    s.add_argument("--queue-depth", type=int, default=64); s.add_argument("--queue-wait", type=float, default=30.0)
    s.add_argument("--kv-early-termination-min-output-tokens", type=int, default=-1,
                   help="end a request that would stall for KV with finish_reason length (finish_detail kv_pressure) once it has "
                        "produced this many tokens; -1 = off: requests stall, never end early")
    s.add_argument("--prefix-cache-entries", type=int, default=0,
                   help="snapshots the prefix cache retains at most (0 = as many as half the KV pool holds); the least recently used goes first")
    s.add_argument("--kv-decode-reserve-chunk", type=int, default=0,
                   help="tokens a request leases beyond its prompt and tops up by when decode reaches them (0 = 16384)")
    s.add_argument("--max-output-tokens", type=int, default=int(os.environ.get("CUTEAFD_MAX_OUTPUT_TOKENS", 0)),
                   help="most output tokens a request may ask for, and what a request that names no limit gets; 0 = bounded by the "
                        "context alone (such a request then gets 256)")
    s.add_argument("--fake-engine", action="store_true", help="serve with the CPU oracle engine (no GPU)")
    s.add_argument("--usage-db", default=""); s.add_argument("--memory-spool", default="", help="file opened at start-up that receives the ledger's state when an allocation fails"); s.add_argument("--kv-format", default="auto", choices=["auto", "bf16", "fp8_ds_mla"])
    s.add_argument("--batch-invariant", action="store_true", default=os.environ.get("CAFD_BATCH_INVARIANT", "0") == "1",
                   help="a row's output bits do not depend on what else is in a decode step (up to 64 rows): kv splits of a fixed "
                        "1024 tokens instead of an even division that fills the GPU, one absorb route for every MLA decode width")
    s.add_argument("--embedding-placement", default="gpu", choices=["gpu", "host"],
                   help="host: the token embedding table stays memory-mapped in host RAM and each step's rows are gathered and uploaded")
    s.add_argument("--host-cache-gib", type=float, default=float(os.environ.get("CUTEAFD_HOST_CACHE_GIB", "4")),
                   help="pinned host memory behind the device prefix cache: evicted snapshots are kept there and restored on a later hit (0 = off)")
    s.add_argument("--loop-abort-run", type=int, default=int(os.environ.get("CUTEAFD_LOOP_ABORT_RUN", 512)),
                   help="end a response (finish_reason length, finish_detail repetition) after this many consecutive "
                        "32-token shingles that repeat a block longer than 256 tokens; 0 = off")
    s.add_argument("--loop-abort-copies", type=int, default=int(os.environ.get("CUTEAFD_LOOP_ABORT_COPIES", 8)),
                   help="verbatim copies of a long block that count as a loop")
    s.add_argument("--loop-fast-span", type=int, default=int(os.environ.get("CUTEAFD_LOOP_FAST_SPAN", 1024)),
                   help="short-cycle rule: tokens the copies after the first must span; 0 = off")
    s.add_argument("--loop-fast-copies", type=int, default=int(os.environ.get("CUTEAFD_LOOP_FAST_COPIES", 8)),
                   help="identical copies of a short unit (1..256 tokens) that count as a loop")
    s.add_argument("--draft-snapshot", default="", help="with --speculator draft-model / block-draft: the small checkpoint (same vocabulary) that drafts")
    s.add_argument("--profile", default="", help="comma-separated host-side profile modes (also $PROFILE): draft-timing, expert-routes, census, step-timing")
    s.add_argument("--profile-dir", default="", help="directory for the files the profile modes append to (default: the working directory)")
    s.add_argument("--speculation-trace", default="", help="JSONL file, one record per decode round (also $SPECULATION_TRACE); "
                                                            "written by a bounded background writer that drops, never blocks")
    s.add_argument("--stall-dump-seconds", type=float, default=0.0,
                   help="write every thread's stack when requests are in flight and the loop has not ticked for this long; 0 = off")
    s.add_argument("--stack-dump-file", default="", help="where SIGUSR1 and stall dumps go (default: stderr)")
    s.add_argument("--prewarm", default="", help="JSON list of decode step geometries: read at start, rewritten at exit; 'auto' = the derived default list")
    s.add_argument("--media-encoder", default="", help="host:port of an encoderd service that holds the media towers (instead of --media)")
    s.add_argument("--media", default="none", choices=["none", "auto", "random"],
                   help="auto: load the vision / audio towers the snapshot bundles; random: small random-init towers")
    s.set_defaults(fn=cmd_serve)

    la = sub.add_parser("launch", help="plan a checkpoint on this box and start one serving process per rank")
    la.add_argument("model", nargs="?", default="")
    la.add_argument("--deployment", default="", help="start this deployment document (from plan --deployment) instead of planning")
    la.add_argument("--run-dir", default="cuteafd-run", help="directory for the deployment document, the per-rank logs and the pid file")
    la.add_argument("--dry-run", action="store_true", help="validate the plan and print the per-rank commands without starting anything")
    la.add_argument("--gpus", type=int, default=8, help="GPUs of the box to plan for")
    la.add_argument("--attention-ranks", type=int, default=1); la.add_argument("--expert-ranks", type=int, default=None)
    la.add_argument("--pool-tokens", type=int, default=None); la.add_argument("--gpu-memory-cap", default="")
    la.add_argument("--kv-pool-size", default="", help="KV pool target as a size per attention GPU (22.5GB, 90GiB) instead of --pool-tokens")
    la.add_argument("--max-context-tokens", type=int, default=None, help="longest context a request may reach")
    la.add_argument("--concurrency", type=int, default=None, help="requests decoded together")
    la.add_argument("--speculator", default=None, type=_speculator, choices=["auto", "off", "mtp"], help="speculative decoding to plan for and serve with")
    la.add_argument("--core-view", default=None, choices=CORE_VIEWS, help="dense-core variant of a multi-core checkpoint (cuteafd-mc.json): the source core, a stored 8- / 6-bit trellis core, or the source core encoded to E4M3 block-128 at load")
    la.add_argument("--decode-lanes", type=int, default=None, choices=[1, 2])
    la.add_argument("--host", default="127.0.0.1", help="address rank 0's HTTP server listens on")
    la.add_argument("--port", type=int, default=8000, help="port of rank 0's HTTP server")
    la.add_argument("--api-key", default=os.environ.get("CUTEAFD_API_KEY", ""), help="bearer key the HTTP server asks for")
    la.add_argument("--master-addr", default="127.0.0.1", help="rendezvous address of the process group")
    la.add_argument("--master-port", type=int, default=29500, help="rendezvous port of the process group")
    la.add_argument("--serve-arg", action="append", default=[], metavar="ARG", help="extra argument handed to every rank's serve command (repeatable)")
    la.set_defaults(fn=cmd_launch)

    st = sub.add_parser("stop", help="end a deployment started by launch")
    st.add_argument("--run-dir", default="cuteafd-run", help="the run directory given to launch")
    st.set_defaults(fn=cmd_stop)

    e = sub.add_parser("expertd", help="expert-rank worker")
    e.add_argument("--snapshot", default=""); e.add_argument("--rank", type=int, default=1); e.add_argument("--world", type=int, default=2)
    e.add_argument("--tcp-port", type=int, default=None,
                   help="serve over the TCP wire protocol instead of joining the box's NVLink group (a worker on another host); 0 = any port")
    e.add_argument("--experts", default="", help="with --tcp-port: first:end of the expert ids this worker holds")
    e.add_argument("--host", default="127.0.0.1", help="with --tcp-port: address to listen on")
    e.add_argument("--device", default="cpu", help="with --tcp-port: device the experts run on")
    e.add_argument("--master-addr", default="127.0.0.1"); e.add_argument("--master-port", type=int, default=29500)
    e.add_argument("--deployment", default="")
    e.set_defaults(fn=cmd_expertd)

    g = sub.add_parser("golden", help="layer-by-layer comparison of the engine against the CPU oracle")
    g.add_argument("--snapshot", default=""); g.add_argument("--preset", default="tiny-moe"); g.add_argument("--tokens", type=int, default=64)
    g.add_argument("--out", default="")
    g.add_argument("--layer-major", default="", metavar="DIR", help="write the oracle's reference dumps of --snapshot into DIR (tokens.bin, "
                   "layerNN.bin, logits.bin) one layer's weights at a time; a run that was interrupted continues after the last finished layer")
    g.add_argument("--windows", type=int, default=4, help="with --layer-major: independent windows of --tokens tokens each")
    g.set_defaults(fn=cmd_golden)

    b = sub.add_parser("bench", help="run the headline benchmark card")
    b.add_argument("--gpus", type=int, default=1); b.add_argument("--steps", type=int, default=128)
    b.add_argument("--warmup", type=int, default=8); b.add_argument("--port", type=int, default=29511)
    b.add_argument("--url", default="", help="run panels against this live server over HTTP instead of the in-process card")
    b.add_argument("--panels", default="quick", help="comma-separated: smoke, cache_exact, lossless, template, tools, speed, sweep, "
                                                       "sustained, agentic, context_load, fidelity; quick = the first five")
    b.add_argument("--sessions", type=int, default=4, help="agentic panel: conversations run side by side")
    b.add_argument("--turns", type=int, default=4, help="agentic panel: turns per conversation")
    b.add_argument("--windows", default="", help="fidelity panel: sealed reference windows (written by `fidelity seal`)")
    b.add_argument("--kl-bar", type=float, default=0.05, help="fidelity panel: largest accepted mean KL")
    b.add_argument("--top1-bar", type=float, default=0.93, help="fidelity panel: smallest accepted top-1 agreement")
    b.add_argument("--fidelity-windows", type=int, default=8, help="fidelity panel: windows scored (8 = the quick set)")
    b.add_argument("--lengths", default="1024,4096,16384,65536", help="context_load panel: prompt lengths in tokens")
    b.add_argument("--vocab", type=int, default=256, help="context_load panel: token ids are drawn below this")
    b.add_argument("--api-key", dest="bench_api_key", default=os.environ.get("CUTEAFD_API_KEY", ""), help="bearer token of the server under test")
    b.add_argument("--max-tokens", type=int, default=64, help="tokens generated per request in the panels")
    b.add_argument("--levels", default="1,4,8", help="concurrency levels of the sweep panel")
    b.add_argument("--seconds", type=float, default=10.0, help="duration of the sustained panel")
    b.add_argument("--concurrency", type=int, default=4, help="streams of the sustained panel")
    b.add_argument("--report-root", default="", help="place a report (report.json, card.svg, card.md) of this run under ROOT/benchmarks/<family>/")
    b.add_argument("--from-json", default="", help="with --report-root: build the report from a saved bench.py result line instead of running")
    b.add_argument("--family", default="", help="family name the report is filed under")
    b.add_argument("--checkpoint", default="", help="checkpoint name the report carries")
    b.add_argument("--hardware", default="", help="hardware layout label of a panel report, e.g. 8gpu-1att-7exp")
    b.add_argument("--profile-name", default="smoke", help="profile label of the report directory")
    b.add_argument("--publish", default="", metavar="ROOT", help="rebuild ROOT/README.md's results table and ROOT/benchmarks/README.md from the reports on disk")
    b.add_argument("--check", action="store_true", help="with --publish: write nothing, exit 1 when the generated blocks are stale")
    b.set_defaults(fn=cmd_bench)

    f = sub.add_parser("fabric", help="NVLink / peer-access report")
    f.add_argument("--json", action="store_true"); f.add_argument("--p2p", action="store_true")
    f.set_defaults(fn=cmd_fabric)

    sub.add_parser("doctor", help="environment checks").set_defaults(fn=cmd_doctor)

    mcp = sub.add_parser("mc", help="multi-core checkpoint repositories (several dense-core variants behind one cuteafd-mc.json)")
    mcp.add_argument("action", choices=["validate", "views"], help="validate: every view's hashes, fingerprint, shared inventory and "
                                                                   "the cross-view rules; views: list the views")
    mcp.add_argument("directory", help="the repository (a snapshot directory)")
    mcp.set_defaults(fn=cmd_mc)
    pw = sub.add_parser("prewarm", help="a decode-graph prewarm list from the speculation trace of an earlier run")
    pw.add_argument("trace", help="JSONL written by serve --speculation-trace")
    pw.add_argument("--out", default="", help="file to write (default: standard output); give it to serve --prewarm")
    pw.add_argument("--top", type=int, default=32, help="how many of the most frequent step geometries to keep")
    pw.set_defaults(fn=cmd_prewarm)
    gw = sub.add_parser("gateway", help="protocol gateway in front of an OpenAI-compatible upstream")
    gw.add_argument("--upstream", default="http://127.0.0.1:8000"); gw.add_argument("--host", default="127.0.0.1")
    gw.add_argument("--port", type=int, default=8080); gw.add_argument("--model-map", default="")
    gw.add_argument("--record", default="", help="append every upstream exchange to this JSONL file")
    gw.add_argument("--replay", default="", help="answer from a recorded JSONL file, never contacting the upstream")
    gw.set_defaults(fn=cmd_gateway)

    q = sub.add_parser("quantize", help="re-encode a snapshot into a serving format (per-role recipe)")
    q.add_argument("src"); q.add_argument("dst")
    for role, default in (("routed_expert", "keep"), ("shared_expert", "keep"), ("dense_ffn", "keep"), ("attention", "keep"),
                          ("indexer", "keep"), ("mtp", "keep")):
        q.add_argument("--" + role.replace("_", "-"), dest=role, default=default, help="target format for this role")
    q.add_argument("--rank", type=int, default=0); q.add_argument("--world", type=int, default=1)
    q.add_argument("--device", default="cpu"); q.add_argument("--seed", type=int, default=0)
    q.add_argument("--hessians", default="", help="directory of <operand>.hessian tensors from a calibration run (EXL3 error feedback)")
    q.add_argument("--merge-only", action="store_true", help="all workers have finished: write the index and the manifest")
    q.set_defaults(fn=cmd_quantize)

    c = sub.add_parser("calibrate", help="collect per-projection input Hessians for quantize --hessians")
    c.add_argument("src"); c.add_argument("dst")
    c.add_argument("--tokens", default="", help="text file of calibration lines (default: random ids)")
    c.add_argument("--rows", type=int, default=2048); c.add_argument("--seq", type=int, default=256)
    c.add_argument("--seed", type=int, default=0); c.add_argument("--dtype", default="f32", choices=("f32", "bf16"))
    c.set_defaults(fn=cmd_calibrate)

    en = sub.add_parser("encoderd", help="media encoder service: the vision / audio towers behind a TCP port")
    en.add_argument("--snapshot", default="", help="checkpoint whose bundled towers are served")
    en.add_argument("--host", default="127.0.0.1", help="address to listen on")
    en.add_argument("--port", type=int, default=0, help="port to listen on (0 = any)")
    en.add_argument("--device", default="cuda:0", help="device the towers run on (falls back to cpu without a GPU)")
    en.add_argument("--hidden", type=int, default=2048, help="embedding width when no snapshot is given")
    en.add_argument("--random", action="store_true", help="small random-init towers for whatever the snapshot lacks")
    en.set_defaults(fn=cmd_encoderd)

    fd = sub.add_parser("fidelity", help="KL / top-1 of a snapshot against sealed reference windows")
    fd.add_argument("action", choices=["seal", "check"], help="seal: compute and store the reference distributions; check: compare a snapshot with them")
    fd.add_argument("snapshot", help="reference snapshot (seal) or snapshot under test (check)")
    fd.add_argument("file", help="sealed window file (.safetensors)")
    fd.add_argument("--windows", type=int, default=16, help="seal: number of windows")
    fd.add_argument("--seq", type=int, default=128, help="seal: tokens per window")
    fd.add_argument("--tokens", default="", help="seal: text file to cut windows from (default: random ids)")
    fd.add_argument("--seed", type=int, default=0, help="seal: seed of the random windows")
    fd.add_argument("--max-kl", type=float, default=0.05, help="check: largest mean KL that passes")
    fd.add_argument("--min-top1", type=float, default=0.9, help="check: smallest top-1 agreement that passes")
    fd.set_defaults(fn=cmd_fidelity)

    u = sub.add_parser("usage", help="request accounting report")
    u.add_argument("--db", default="usage.sqlite"); u.add_argument("--hours", type=float, default=24.0)
    u.set_defaults(fn=cmd_usage)
    return ap


# Configuration key -> flag destination, where the two are not the same word.
_CONFIG_DEST = {"HTTP_QUEUE_DEPTH": "queue_depth", "HTTP_QUEUE_WAIT": "queue_wait"}


def serve_args_from_config(file_config: dict[str, str], already: list[str]) -> list[str]:
    """Configuration keys that are flags of ``serve`` but not of ``launch`` (MAX_OUTPUT_TOKENS, BATCH_INVARIANT,
    DRAFT_LENGTH, PROFILE, ...) become arguments of every rank's serve command; a flag the launch line already hands to
    the ranks (its own or a ``--serve-arg``) wins over the file."""
    subs = next(x for x in build_parser()._actions if isinstance(x, argparse._SubParsersAction))
    serve = {x.dest: x for x in subs.choices["serve"]._actions if x.option_strings}
    launch = {x.dest for x in subs.choices["launch"]._actions if x.option_strings or x.dest == "model"}
    given = {t.split("=", 1)[0] for t in already if t.startswith("--")}
    out: list[str] = []
    for key, raw in file_config.items():
        dest = _CONFIG_DEST.get(key, key.lower())
        act = serve.get(dest)
        if act is None or dest in launch or key == "MODEL" or any(o in given for o in act.option_strings):
            continue
        flag = max(act.option_strings, key=len)
        if isinstance(act, argparse._StoreTrueAction):
            if raw.strip().lower() in ("1", "on", "true", "yes"):
                out.append(flag)
            continue
        val = act.type(raw) if act.type is not None else raw
        if act.choices is not None and val not in act.choices:
            print(f"config: {key}={raw} is not one of {sorted(map(str, act.choices))}", file=sys.stderr)
            raise SystemExit(2)
        out += [flag, raw]
    return out


def apply_config(ap: argparse.ArgumentParser, a: argparse.Namespace, argv: list[str]) -> None:
    """Configuration keys become the values of the sub-command's flags of the same name (MODEL also names the
    ``--snapshot`` of serve / expertd / golden); a flag given on the command line wins over the file, ``--set`` wins
    over the file's own lines.  Keys the sub-command has no flag for are left for it to read from ``a.file_config``."""
    subs = next(x for x in ap._actions if isinstance(x, argparse._SubParsersAction))
    sp = subs.choices[a.cmd]
    given = {t.split("=", 1)[0] for t in argv if t.startswith("--")}
    by_dest = {x.dest: x for x in sp._actions if x.option_strings or x.dest == "model"}
    for key, raw in a.file_config.items():
        dests = [_CONFIG_DEST.get(key, key.lower())] + (["snapshot"] if key == "MODEL" else [])
        for d in dests:
            act = by_dest.get(d)
            if act is None or any(o in given for o in act.option_strings):
                continue
            if not act.option_strings and getattr(a, d, None) not in (None, ""):
                continue                                         # a positional given on the command line
            if isinstance(act, (argparse._StoreTrueAction, argparse._StoreFalseAction)):
                val = raw.strip().lower() in ("1", "on", "true", "yes")
            else:
                val = act.type(raw) if act.type is not None else raw
                if act.choices is not None and val not in act.choices:
                    print(f"config: {key}={raw} is not one of {sorted(map(str, act.choices))}", file=sys.stderr)
                    raise SystemExit(2)
            setattr(a, d, val)


def main(argv: list[str] | None = None) -> int:
    ap = build_parser()
    argv = list(sys.argv[1:] if argv is None else argv)
    a = ap.parse_args(argv)
    a.file_config = load_config_file(a.config, a.set, CONFIG_KEYS) if (a.config or a.set) else {}
    if a.file_config:
        apply_config(ap, a, argv)
    return a.fn(a)


if __name__ == "__main__":
    raise SystemExit(main())
