"""``cuteafd expertd``: one expert-rank worker process.

Joins the NCCL group of a deployment, maps the symmetric exchange buffers, loads the routed
experts it owns (from a snapshot, or random weights for benchmarks) and serves announced steps
until the attention rank says stop.  Counterpart:
rust/crates/cuteafd-daemon/src/shared/experts/service.rs:22-135, service/local.rs:278.
"""
from __future__ import annotations

import json
import os


def run_tcp_worker(args) -> int:
    """Off-box worker: serves experts [first, end) of a snapshot over the wire protocol (``parallel/wire.py``).  On a
    CUDA ``--device`` the routed FFN runs on the tcgen05 expert-grouped GEMMs (``wire.cuda_compute``); on ``cpu`` it is
    plain tensor code (the oracle's arithmetic).  The plan hash covers the model name and the expert range, so an
    attention rank configured for another split is refused at the handshake."""
    import time

    import torch

    from ..loader.load import load_params
    from ..parallel import wire
    lo, hi = (int(v) for v in args.experts.split(":"))
    cfg, params = load_params(args.snapshot, dtype=torch.bfloat16, device=args.device, only=".mlp.experts.")
    stacks: dict[int, tuple] = {}

    def stack_of(layer: int):
        if layer not in stacks:
            m = f"model.layers.{layer}.mlp.experts."
            stacks[layer] = tuple(torch.stack([params[f"{m}{e}.{n}_proj.weight"] for e in range(lo, hi)]).contiguous()
                                  for n in ("gate", "up", "down"))
        return stacks[layer]
    plan = wire.plan_hash({"model": cfg.name, "experts": cfg.num_experts, "range": [lo, hi]})
    on_gpu = str(args.device).startswith("cuda")
    compute = wire.cuda_compute(stack_of, lo, args.device, cfg.expert_ffn) if on_gpu else wire.reference_compute(stack_of, lo)
    srv = wire.ExpertServer(compute, plan, args.host, args.tcp_port).start()
    print(f"expert worker for experts [{lo}, {hi}) of {cfg.name} on {args.host}:{srv.port}", flush=True)
    try:
        while True:
            time.sleep(3600)
    except KeyboardInterrupt:
        srv.stop()
    return 0


def run_expertd(args) -> int:
    if getattr(args, "tcp_port", None) is not None:
        return run_tcp_worker(args)
    import torch
    import torch.distributed as dist

    from ..config import PRESETS
    from ..parallel.afd import build_afd
    os.environ.setdefault("MASTER_ADDR", args.master_addr)
    os.environ.setdefault("MASTER_PORT", str(args.master_port))
    dep = json.load(open(args.deployment)) if args.deployment else {}
    local = int(os.environ.get("LOCAL_RANK", args.rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", rank=args.rank, world_size=args.world, device_id=dev)
    params = None
    if args.snapshot:
        from ..loader.load import load_params
        cfg, params = load_params(args.snapshot, dtype=torch.bfloat16, only=".mlp.experts.")
    else:
        cfg = PRESETS[dep.get("model", "qwen3-30b-a3b")]()
    h = build_afd(cfg, dev, args.rank, args.world, max_tokens=dep.get("prefill_rows", 8192), max_seqs=dep.get("decode_rows", 64),
                  num_pages=2, pages_per_seq=1, params=params)
    if h.worker is None:
        raise SystemExit("expertd must not be rank 0 (rank 0 is the attention rank)")
    h.worker.serve()
    dist.barrier()
    dist.destroy_process_group()
    return 0
