"""Multi-GPU MoE dispatch -> expert -> combine microbenchmark (attention rank GPU 0, experts
expert-parallel over the other GPUs), with the NCCL all-to-all + cuBLAS baseline twin.

    python -m torch.distributed.run --nnodes=1 --nproc-per-node 4 --master-addr 127.0.0.1 --master-port 29544 \
        -m cuteafd_b200.bench.moe_afd_bench --tokens 1,16,128,1024,8192 --hidden 7168 --ffn 2048 --experts 256 \
        --top-k 8 --scoring sigmoid --fp8

Fused path: plan + dispatch kernels store rows into the owners' slabs over NVLink peer memory,
the owners' grouped tcgen05 GEMMs (bf16 or block-scaled E4M3) run fc1/SwiGLU and fc2, the fc2
epilogue stores (token, slot) rows into rank 0's combine buffer, rank 0 reduces.  Time = CUDA
events on rank 0 from the first dispatch kernel to the end of the combine kernel, max over ranks of
the per-rank means.  Roofline target = max(expert FLOPs / measured GEMM peak on the busiest expert
rank, bytes leaving rank 0 / 770 GB/s); the same bytes come back, in the other direction.

Baseline: rows sorted by owner on rank 0, ``all_to_all_single`` out, one cuBLAS GEMM triple per
expert, ``all_to_all_single`` back, index-add on rank 0 (bf16).
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.distributed as dist

from ..ops import kernels as K
from ..parallel.afd import ExpertWorker, RemoteExchange, SymLayout, SymmetricHeap
from ..parallel.moe_exchange import ExchangeGeometry, pick_tile_rows
from ..quant import codecs
from .microbench import peaks

NVLINK_GBS = 770.0


def _rand_w(E, r, c, dev, g):
    w = torch.empty(E, r, c, dtype=torch.bfloat16, device=dev)
    w.normal_(0.0, 0.02, generator=g)
    return w


def _quant_stack(w):
    qs = [codecs.fp8_quant_block128(w[e].float()) for e in range(w.shape[0])]
    return torch.stack([q for q, _ in qs]).contiguous(), torch.stack([s for _, s in qs]).contiguous()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", default="1,16,128,1024,8192")
    ap.add_argument("--hidden", type=int, default=7168); ap.add_argument("--ffn", type=int, default=2048)
    ap.add_argument("--experts", type=int, default=256); ap.add_argument("--top-k", type=int, default=8)
    ap.add_argument("--scoring", default="sigmoid"); ap.add_argument("--groups", type=int, default=8)
    ap.add_argument("--topk-groups", type=int, default=4)
    ap.add_argument("--fp8", action="store_true"); ap.add_argument("--iters", type=int, default=10)
    ap.add_argument("--warm", type=int, default=3); ap.add_argument("--baseline", action="store_true")
    ap.add_argument("--wave-tokens", type=int, default=4096, help="steps above this many tokens are exchanged in waves (0 = off)")
    a = ap.parse_args()
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    local = int(os.environ.get("LOCAL_RANK", rank))
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev)
    Ts = [int(t) for t in a.tokens.split(",")]
    H, I, E, k = a.hidden, a.ffn, a.experts, a.top_k
    n_exp = world - 1
    geo = ExchangeGeometry(H, I, E, k, max(Ts), n_exp, wave_tokens=a.wave_tokens if max(Ts) > a.wave_tokens > 0 else 0)
    lay = SymLayout.build(geo, 1)
    heap = SymmetricHeap(lay.total, dev)
    pk = peaks()
    route_kw = dict(scoring=a.scoring, num_groups=a.groups if a.scoring == "sigmoid" else 1,
                    topk_groups=a.topk_groups if a.scoring == "sigmoid" else 1)
    g = torch.Generator(device=dev).manual_seed(rank)
    results = []
    if rank == 0:
        ex = RemoteExchange(geo, heap, lay, 1, 0)
        epoch = ex.epoch
    else:
        lo, hi = geo.rank_experts(rank - 1)
        wg, wu, wd = _rand_w(hi - lo, I, H, dev, g), _rand_w(hi - lo, I, H, dev, g), _rand_w(hi - lo, H, I, dev, g)
        weights = [(wg, wu, wd)]
        if a.fp8:
            weights = [(_quant_stack(wg), _quant_stack(wu), _quant_stack(wd))]
        worker = ExpertWorker(None, weights, heap, lay, geo, rank)
        epoch = worker.epoch
    dist.barrier()
    for T in Ts:
        tile = pick_tile_rows(min(T, geo.region().max_tokens), k, E)
        if rank == 0:
            x = torch.randn(T, H, device=dev, generator=g).bfloat16()
            res = torch.randn(T, H, device=dev, generator=g).bfloat16()
            logits = torch.randn(T, E, device=dev, generator=g)
            out = torch.empty(T, H, dtype=torch.bfloat16, device=dev)
        times = []
        for it in range(a.warm + a.iters):
            s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            if rank == 0:
                K.bump_epoch(epoch)
            s.record()
            if rank == 0:
                ex.forward(x, logits, route_kw, None, None, None, out, residual=res)
            else:
                worker._step(T)              # bumps its own epoch
            e.record()
            torch.cuda.synchronize()
            if it >= a.warm:
                times.append(s.elapsed_time(e))
            dist.barrier()
        st = K.read_status()
        t = torch.tensor([sum(times) / len(times), float(st)], dtype=torch.float64, device=dev)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t[0])
        flops = 2.0 * T * k * 3 * H * I
        link_bytes = T * k * H * 2.0                           # rows leaving rank 0 (the same amount returns)
        peak = pk["bf16_tflops"] * (2.0 if a.fp8 else 1.0) * 1e12
        # expert weights the busiest rank must stream from HBM: its active experts, each once
        per_rank = -(-E // n_exp)
        active = min(per_rank, T * k)
        w_bytes = active * 3 * H * I * (1.0 if a.fp8 else 2.0)
        target_ms = max(flops / n_exp / peak, link_bytes / (NVLINK_GBS * 1e9), w_bytes / (pk["hbm_gbs"] * 1e9)) * 1e3
        r = {"case": f"moe_afd T={T} H={H} I={I} E={E} k={k} ep={n_exp} {'fp8' if a.fp8 else 'bf16'} tile={tile} waves={len(geo.waves(T))}", "ms": round(ms, 4),
             "nvlink_gbs_each_way": round(link_bytes / ms / 1e6, 1), "tflops": round(flops / ms / 1e9, 1),
             "roofline_target_ms": round(target_ms, 4), "roofline_frac": round(target_ms / ms, 3), "status": int(t[1]), "of": pk["kind"]}
        results.append(r)
        if rank == 0:
            print(json.dumps(r), flush=True)
        # ---- NCCL + cuBLAS twin ---------------------------------------------------------------------
        if a.baseline:
            ms_b = _baseline(rank, world, dev, T, H, I, E, k, geo, a, (x, logits) if rank == 0 else None,
                             None if rank == 0 else (wg, wu, wd, lo, hi))
            if rank == 0:
                print(json.dumps({"case": f"nccl+cublas T={T} ep={n_exp} bf16", "ms": round(ms_b, 4), "speedup_of_fused": round(ms_b / ms, 2)}), flush=True)
    dist.barrier()
    dist.destroy_process_group()


def _baseline(rank, world, dev, T, H, I, E, k, geo, a, att_in, exp_in) -> float:
    from ..ref import ops as R
    times = []
    for it in range(a.warm + a.iters):
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        send_counts = torch.zeros(world, dtype=torch.int64, device=dev)
        if rank == 0:
            x, logits = att_in
            idx, w = R.route_topk(logits, k, a.scoring)
            flat = idx.reshape(-1).long()
            order = torch.argsort(flat, stable=True)
            owners = torch.bucketize(flat[order], torch.tensor([geo.rank_experts(r)[1] for r in range(world - 1)], device=dev), right=True)
            send_counts[1:] = torch.bincount(owners, minlength=world - 1)
            rows = x[(order // k)]
            eids = flat[order].to(torch.int32)
        recv_counts = torch.empty_like(send_counts)
        dist.all_to_all_single(recv_counts, send_counts)
        sc, rc = send_counts.tolist(), recv_counts.tolist()
        n_in = int(sum(rc))
        rows_in = torch.empty(n_in, H, dtype=torch.bfloat16, device=dev)
        eid_in = torch.empty(n_in, dtype=torch.int32, device=dev)
        dist.all_to_all_single(rows_in, rows if rank == 0 else torch.empty(0, H, dtype=torch.bfloat16, device=dev), rc, sc)
        dist.all_to_all_single(eid_in, eids if rank == 0 else torch.empty(0, dtype=torch.int32, device=dev), rc, sc)
        y = torch.empty_like(rows_in)
        if rank != 0 and n_in:
            wg, wu, wd, lo, hi = exp_in
            for ex in torch.unique(eid_in).tolist():
                m = eid_in == ex
                h = torch.nn.functional.silu(rows_in[m] @ wg[ex - lo].T) * (rows_in[m] @ wu[ex - lo].T)
                y[m] = h @ wd[ex - lo].T
        back = torch.empty(int(sum(sc)), H, dtype=torch.bfloat16, device=dev)
        dist.all_to_all_single(back, y, sc, rc)
        if rank == 0:
            out = torch.zeros(T, H, dtype=torch.float32, device=dev)
            out.index_add_(0, order // k, back.float() * w.reshape(-1)[order][:, None])
        e.record()
        torch.cuda.synchronize()
        if it >= a.warm:
            times.append(s.elapsed_time(e))
        dist.barrier()
    t = torch.tensor([sum(times) / len(times)], dtype=torch.float64, device=dev)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t[0])


if __name__ == "__main__":
    main()
