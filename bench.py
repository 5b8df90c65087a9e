#!/usr/bin/env python
"""Headline benchmark: Qwen3-30B-A3B-shaped MoE, bf16, random init, synthetic token-id prompts.

Workload (the reference's Qwen3 release card: cold 8K prefill, then decode sweeps): 8192-token random prompts, then greedy
decode at concurrency 1 / 8 / 32.  Layout: one GPU runs everything; two GPUs = one attention rank + one expert
rank; four and eight GPUs = two data-parallel attention replicas in front of two / six expert ranks (experts
partitioned by id).  A "step" is one decode step of the concurrency-8 batch; ``--steps`` steps are timed on the
device with CUDA events after ``--warmup`` untimed steps, max over ranks.  Prefill tok/s, TTFT and the other
concurrency levels ride along in ``extra``.  With eight GPUs the same card is also run on the DeepSeek-V3 shape
(MLA attention, E4M3 block-scaled experts, 2 attention + 6 expert GPUs) and reported under ``extra.dsv3_*``.

    python bench.py                      # one GPU
    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 \
        --master-port 29511 bench.py --gpus 4
    python bench.py --impl reference     # the unmodified reference, when it can be installed
"""
from __future__ import annotations

import argparse
import json
import os
import sys
import time

REPO = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, REPO)

# Published reference card closest to this configuration (Qwen 3.8 Flash Next EXL3, one RTX PRO
# 6000, MTP x3): C1 / C8 / C16 decode tok/s, 8K prefill tok/s, TTFT seconds.
PUBLISHED = {"c1": 199.2, "c8": 504.1, "c16": 734.6, "prefill_tok_s": 8646.0, "ttft_s": 0.947}


def reference_arm() -> None:
    """The reference is a Rust + CUDA (sm_120/sm_121) engine whose kernel submodule is absent and
    whose Python package does not install offline; there is nothing runnable to time."""
    why = ("reference not installable offline: its source tree has no pyproject/setup.py at its root, "
           "python/ fails metadata generation without its index-only dependencies, the Rust workspace needs "
           "cargo + crates.io, and third_party/sparkinfer (all hot kernels) is an empty submodule")
    ref_dir = os.path.join(REPO, "baseline", "_ref")
    if os.path.isdir(ref_dir) and os.listdir(ref_dir):
        why = "baseline/_ref holds no runnable engine: " + why
    print(json.dumps({"impl": "reference", "unavailable": why}))


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=128)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--prompt-len", type=int, default=8192)
    ap.add_argument("--levels", default="1,8,32")
    ap.add_argument("--layers", type=int, default=0, help="debug only: fewer layers (marks the run invalid)")
    ap.add_argument("--no-graphs", action="store_true")
    ap.add_argument("--config", default="qwen3", choices=["qwen3", "dsv3"],
                    help="qwen3 = the headline Qwen3-30B-A3B bf16 card (with 8 GPUs the DeepSeek-V3 card follows it); dsv3 = only "
                         "the DeepSeek-V3 shape: MLA attention replicas, E4M3 block-scaled experts on the other GPUs (needs 8 GPUs)")
    ap.add_argument("--attention-ranks", type=int, default=0,
                    help="data-parallel attention replicas of the disaggregated layout (0 = 1 on two GPUs, 2 on four or more)")
    ap.add_argument("--no-dsv3", action="store_true", help="with 8 GPUs: skip the DeepSeek-V3 card that follows the headline card")
    ap.add_argument("--prefill-chunk", type=int, default=0)
    ap.add_argument("--parallelism", default="auto", choices=["auto", "afd", "tp"],
                    help="layout on more than one GPU: afd = attention on GPU 0, routed experts on the others; tp = attention "
                         "heads split over all GPUs with the residual rows sharded and every rank running the FFN of its "
                         "own rows (experts replicated); auto = afd")
    args = ap.parse_args()
    if args.impl == "reference":
        reference_arm()
        return

    import torch
    import torch.distributed as dist

    from cuteafd_b200 import qwen3_30b_a3b
    from cuteafd_b200.bench.card import run_card
    from cuteafd_b200.bench.clocks import ClockSampler

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    assert world == args.gpus, f"--gpus {args.gpus} but WORLD_SIZE={world}"
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    warmup = max(3, args.warmup)
    levels = tuple(int(x) for x in args.levels.split(","))
    headline = 8 if 8 in levels else levels[-1]
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)

    def log(msg: str) -> None:
        if rank == 0:
            print(f"[bench] {msg}", file=sys.stderr, flush=True)

    pages_per_seq = (args.prompt_len + 2 * (args.steps + warmup) + 128) // 64 + 2
    num_pages = max(levels) * pages_per_seq + 8 * max(levels) + 64

    def run_config(name: str):
        """Build the deployment of one model configuration, run the card on it, tear it down.  Returns (cfg, card result
        or None on ranks that do not drive a card, parallelism string, clocks summary)."""
        cfg = qwen3_30b_a3b()
        if name == "dsv3":
            from cuteafd_b200 import deepseek_v3
            cfg = deepseek_v3().replace(mtp_layers=0)
            assert world > 2, "the DeepSeek-V3 shape needs expert ranks"
        if args.layers:
            cfg = cfg.replace(num_layers=args.layers)
        handle, gen, sync, replica, replicas = None, None, None, 0, 1
        mode = "afd" if args.parallelism == "auto" else args.parallelism
        t0 = time.time()
        if world > 1 and mode == "tp":
            assert name == "qwen3", "the tensor-parallel layout serves the GQA family"
            from cuteafd_b200.models.gqa_moe import GqaMoeWeights
            from cuteafd_b200.models.tp_gqa import TpGqaMoeEngine
            from cuteafd_b200.runtime.generate import Generator
            from cuteafd_b200.runtime.native import make_pool
            W = GqaMoeWeights.random_init(cfg, dev, seed=0)
            eng = TpGqaMoeEngine(cfg, W, num_pages, max_tokens=args.prompt_len, max_seqs=max(levels))
            gen = Generator(eng, make_pool(num_pages), pages_per_seq, max(levels), prefill_chunk=args.prompt_len,
                            use_graphs=not args.no_graphs)
            torch.cuda.synchronize()
            dist.barrier()
            sync = dist.barrier
            parallelism = (f"tp{world}: attention heads split over {world} GPUs, residual rows sharded, FFN of the owned rows on "
                           f"every rank (experts replicated), fused reduce-scatter / all-gather kernels over NVLink")
        elif world > 1:
            from cuteafd_b200.parallel.afd import build_afd
            A = args.attention_ranks or (1 if world < 4 else 2)
            handle = build_afd(cfg, dev, rank, world, max_tokens=args.prompt_len, max_seqs=max(levels),
                               num_pages=num_pages, pages_per_seq=pages_per_seq, use_graphs=not args.no_graphs,
                               expert_format="fp8" if name == "dsv3" else "bf16",
                               prefill_chunk=args.prefill_chunk or None, n_attention=A)
            gen, parallelism, replica, replicas = handle.generator, handle.parallelism, handle.replica, handle.n_replicas
            torch.cuda.synchronize()
            dist.barrier()
            log(f"{name}: {parallelism} ready in {time.time()-t0:.1f}s, {torch.cuda.memory_allocated()/2**30:.1f} GiB on attention rank 0")
            if handle.worker is not None:
                handle.worker.serve()            # returns when attention rank 0 sends STOP
        else:
            from cuteafd_b200.models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
            from cuteafd_b200.runtime.generate import Generator
            from cuteafd_b200.runtime.native import make_pool
            W = GqaMoeWeights.random_init(cfg, dev, seed=0)
            kv = KvCache(cfg, num_pages, dev)
            eng = GqaMoeEngine(cfg, W, kv, max_tokens=args.prompt_len, max_seqs=max(levels))
            gen = Generator(eng, make_pool(num_pages), pages_per_seq, max(levels), prefill_chunk=args.prompt_len,
                            use_graphs=not args.no_graphs)
            torch.cuda.synchronize()
            log(f"model + KV ready in {time.time()-t0:.1f}s, {torch.cuda.memory_allocated()/2**30:.1f} GiB")
            parallelism = "attention+experts on 1 GPU"
        res, clocks = None, None
        if gen is not None:                      # attention ranks drive the card
            g = torch.Generator().manual_seed(1)
            prompts = [torch.randint(0, cfg.vocab_size, (args.prompt_len,), generator=g).tolist() for _ in range(max(levels))]
            with ClockSampler(local) as clk:
                res = run_card(gen, prompts, levels, args.steps, warmup, sync=sync, log=log, replica=replica, n_replicas=replicas)
            clocks = clk.summary()
            if handle is not None:
                if replica == 0:
                    handle.shutdown()
                else:                            # the stop message replica 0 just sent
                    dist.broadcast(gen.engine.ctrl, src=0)
        if world > 1:
            dist.barrier()
        del gen, handle
        import gc
        gc.collect()
        torch.cuda.empty_cache()
        return cfg, res, parallelism, clocks

    def card_extra(res, prefix: str = "") -> dict:
        extra = {f"{prefix}decode_tok_s_c{c}": round(d.tok_s, 1) for c, d in res.decode.items()}
        extra.update({f"{prefix}e2e_decode_tok_s_c{c}": round(d.e2e_tok_s, 1) for c, d in res.decode.items()})
        extra.update({f"{prefix}prefill_tok_s_8k": round(res.prefill_tok_s, 1), f"{prefix}ttft_s_8k": round(res.ttft_s, 4)})
        return extra

    cfg, res, parallelism, clocks = run_config(args.config)
    valid = not args.layers
    out = None
    if rank == 0 and res is not None:
        r = res.decode[headline]
        extra = card_extra(res)
        if args.config == "qwen3":
            extra["vs_published"] = {"c1": round(res.decode[1].tok_s / PUBLISHED["c1"], 2) if 1 in res.decode else None,
                                     "prefill": round(res.prefill_tok_s / PUBLISHED["prefill_tok_s"], 2),
                                     "ttft": round(PUBLISHED["ttft_s"] / res.ttft_s, 2)}
        out = {
            "metric": f"decode tok/s @ conc {headline} (8K-token prompts; conc 1/8/32, 8K-prefill tok/s and TTFT in extra)",
            "value": round(r.tok_s, 2), "unit": "tok/s", "n_gpus": args.gpus, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(r.ms_per_step, 4), "higher_is_better": True, "scaling": "strong",
            "vs_baseline": round(r.tok_s / PUBLISHED["c8"], 3) if headline == 8 and args.config == "qwen3" else None,
            "dtype": "bf16" if args.config == "qwen3" else "fp8 experts and, at decode, fp8 q_b / o / shared-expert projections (E4M3, 128x128 weight / 1x128 activation scales); MLA attention math, q_a / kv_a and prompt chunks in bf16", "data": "synthetic (uniform random token ids, N(0,0.02) random-init weights)",
            "config": {"model": cfg.name + ("" if valid else f"-{cfg.num_layers}layers-INVALID"),
                       "global_batch": headline, "seq_len": args.prompt_len, "parallelism": parallelism,
                       "l2": "inputs larger than L2 (each step streams GBs of weights and KV)",
                       "timing": "CUDA events around K graph replays, max over ranks"},
            "clocks": clocks,
            "e2e": {"value": round(r.e2e_tok_s, 2), "unit": "tok/s", "h2d_bytes_per_step": r.h2d_bytes_per_step,
                    "d2h_bytes_per_step": r.d2h_bytes_per_step, "ms_per_step": round(r.e2e_ms_per_step, 4)},
            "gpu_launches": r.launches_per_step * args.steps,
            "extra": extra,
        }
    # The named target deployment rides along when the box has the GPUs for it: DeepSeek-V3 shape, E4M3 block-scaled experts,
    # two attention GPUs + six expert GPUs (its closest published card: GLM 5.3, 2 coordinators + 6 expert boxes).
    if world == 8 and args.config == "qwen3" and not args.no_dsv3 and args.parallelism != "tp":
        try:
            dcfg, dres, dpar, dclk = run_config("dsv3")
            if rank == 0 and dres is not None and out is not None:
                out["extra"].update(card_extra(dres, "dsv3_"))
                out["extra"]["dsv3_config"] = {"model": dcfg.name + ("" if valid else f"-{dcfg.num_layers}layers-INVALID"),
                                               "parallelism": dpar, "dtype": "fp8 experts and, at decode, fp8 q_b / o / shared-expert projections (E4M3, 128x128 weight / 1x128 activation scales); MLA attention math, q_a / kv_a and prompt chunks in bf16",
                                               "clocks": dclk,
                                               "vs_published_glm53_2rtx_6spark": {
                                                   "c1": round(dres.decode[1].tok_s / 39.3, 2) if 1 in dres.decode else None,
                                                   "c8": round(dres.decode[8].tok_s / 86.8, 2) if 8 in dres.decode else None,
                                                   "prefill": round(dres.prefill_tok_s / 3331.0, 2), "ttft": round(2.46 / dres.ttft_s, 2)}}
        except Exception as e:                   # the headline line is still printed
            if rank == 0 and out is not None:
                out["extra"]["dsv3_error"] = f"{type(e).__name__}: {e}"
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    if rank == 0 and out is not None:
        print(json.dumps(out), flush=True)


if __name__ == "__main__":
    main()
