"""A few eager decode steps of a shortened Qwen3-30B-A3B-shape (or, with ``--config dsv3``, DeepSeek-V3-shape) model,
bracketed by cudaProfilerStart/Stop, as a target for per-kernel launch lists:

    python -m cuteafd_b200.bench.decode_profile --concurrency 8 --context 8192 --layers 2
    ncu --metrics gpu__time_duration.sum --clock-control none --profile-from-start off --csv --log-file launches.csv \
        python -m cuteafd_b200.bench.decode_profile --concurrency 8

Every layer of the full model launches the same kernels on the same shapes, so two layers give the per-layer
breakdown while holding only a few GB on the device.
"""
from __future__ import annotations

import argparse

import torch

from .. import deepseek_v3, qwen3_30b_a3b
from ..models.gqa_moe import GqaMoeEngine, GqaMoeWeights, KvCache
from ..runtime.generate import Generator
from ..runtime.native import make_pool


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--concurrency", type=int, default=8)
    ap.add_argument("--context", type=int, default=8192)
    ap.add_argument("--layers", type=int, default=2)
    ap.add_argument("--steps", type=int, default=3)
    ap.add_argument("--config", default="qwen3", choices=["qwen3", "dsv3"])
    a = ap.parse_args()
    dev = torch.device("cuda:0")
    pps = a.context // 64 + 4
    pages = a.concurrency * pps + 8
    if a.config == "dsv3":
        # one dense layer + the rest MoE (all 256 routed experts of a layer are 22.5 GB in bf16: keep --layers small)
        from ..models.mla_moe import LatentCache, MlaMoeEngine, MlaMoeWeights
        cfg = deepseek_v3().replace(num_layers=a.layers, first_dense_layers=1, mtp_layers=0)
        W = MlaMoeWeights.random_init(cfg, dev)
        eng = MlaMoeEngine(cfg, W, LatentCache(cfg, pages, dev), max_tokens=a.context, max_seqs=a.concurrency)
    else:
        cfg = qwen3_30b_a3b().replace(num_layers=a.layers)
        W = GqaMoeWeights.random_init(cfg, dev)
        eng = GqaMoeEngine(cfg, W, KvCache(cfg, pages, dev), max_tokens=a.context, max_seqs=a.concurrency)
    gen = Generator(eng, make_pool(pages), pps, a.concurrency, prefill_chunk=a.context, use_graphs=False)
    g = torch.Generator().manual_seed(0)
    seqs, last = [], []
    for _ in range(a.concurrency):
        s = gen.table.new()
        last.append(gen.prefill(s, torch.randint(0, cfg.vocab_size, (a.context,), generator=g).tolist()))
        seqs.append(s)
    torch.cuda.synchronize()
    torch.cuda.profiler.start()
    for _ in range(a.steps):
        last = gen.decode(seqs, last)
    torch.cuda.synchronize()
    torch.cuda.profiler.stop()
    print("done", last)


if __name__ == "__main__":
    main()
