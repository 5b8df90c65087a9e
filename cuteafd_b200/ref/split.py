"""Whole-versus-split oracle: the tiny decoder run once on one rank and once as one attention
rank plus expert ranks exchanging activations over a ``torch.distributed`` group (gloo on CPU).

The split run is the CPU model of attention/FFN disaggregation with experts partitioned by id:
the attention rank broadcasts (rows, routes, gate weights), every expert rank returns the
weighted per-(row, slot) output of the experts it owns, and the attention rank sums the slots
in slot order.  A slot is non-zero on exactly one rank, so the cross-rank sum is exact and the
split logits match the whole run bit for bit.  The reference tests its exchange the same way
without hardware: loopback transports and synthetic executors
(rust/crates/cuteafd-transport/src/synthetic.rs, rust/crates/cuteafd-transport/src/lib.rs:140-170).
"""
from __future__ import annotations

import os
import tempfile

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from ..config import ModelConfig
from . import ops
from .model import RefDecoder, init_weights

OP_STOP, OP_MOE = 0, 1


def expert_range(num_experts: int, expert_ranks: int, r: int) -> tuple[int, int]:
    """Contiguous expert ids owned by expert rank r (uneven splits give the first ranks one more)."""
    base, rem = divmod(num_experts, expert_ranks)
    lo = r * base + min(r, rem)
    return lo, lo + base + (1 if r < rem else 0)


def _attention_rank(cfg: ModelConfig, params, prompts: torch.Tensor, steps: int, out_path: str) -> None:
    H, k = cfg.hidden, cfg.top_k

    def moe_fn(layer: int, x: torch.Tensor, idx: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
        T = x.shape[0]
        dist.broadcast(torch.tensor([OP_MOE, layer, T], dtype=torch.int64), src=0)
        dist.broadcast(x.contiguous(), src=0)
        dist.broadcast(idx.contiguous(), src=0)
        dist.broadcast(w.contiguous(), src=0)
        parts = torch.zeros(T, k, H, dtype=torch.float32)
        dist.reduce(parts, dst=0, op=dist.ReduceOp.SUM)
        return parts

    model = RefDecoder(cfg, params, moe_fn=moe_fn)
    toks, logits = model.generate(prompts, steps)
    dist.broadcast(torch.tensor([OP_STOP, 0, 0], dtype=torch.int64), src=0)
    torch.save({"tokens": toks, "logits": logits}, out_path)


def _expert_rank(cfg: ModelConfig, params, rank: int, world: int) -> None:
    lo, hi = expert_range(cfg.num_experts, world - 1, rank - 1)
    model = RefDecoder(cfg, params)
    dtype = params["model.embed_tokens.weight"].dtype
    while True:
        head = torch.zeros(3, dtype=torch.int64)
        dist.broadcast(head, src=0)
        op, layer, T = (int(v) for v in head)
        if op == OP_STOP:
            return
        x = torch.empty(T, cfg.hidden, dtype=dtype)
        idx = torch.empty(T, cfg.top_k, dtype=torch.int32)
        w = torch.empty(T, cfg.top_k, dtype=torch.float32)
        dist.broadcast(x, src=0)
        dist.broadcast(idx, src=0)
        dist.broadcast(w, src=0)
        parts = ops.moe_forward(x, idx, w, *model.expert_stack(layer, lo, hi), expert_base=lo)
        dist.reduce(parts, dst=0, op=dist.ReduceOp.SUM)


def _worker(rank: int, world: int, cfg: ModelConfig, seed: int, prompts: torch.Tensor, steps: int,
            init_file: str, out_path: str) -> None:
    torch.set_num_threads(1)
    dist.init_process_group("gloo", init_method=f"file://{init_file}", rank=rank, world_size=world)
    params = init_weights(cfg, seed)
    with torch.no_grad():
        if rank == 0:
            _attention_rank(cfg, params, prompts, steps, out_path)
        else:
            _expert_rank(cfg, params, rank, world)
    dist.barrier()
    dist.destroy_process_group()


def run_split(cfg: ModelConfig, prompts: torch.Tensor, steps: int, expert_ranks: int = 2, seed: int = 0):
    """Run the split decode as ``1 + expert_ranks`` gloo processes; returns (tokens, logits)."""
    world = 1 + expert_ranks
    with tempfile.TemporaryDirectory() as d:
        init_file, out = os.path.join(d, "rdzv"), os.path.join(d, "out.pt")
        mp.spawn(_worker, args=(world, cfg, seed, prompts, steps, init_file, out), nprocs=world, join=True)
        r = torch.load(out)
    return r["tokens"], r["logits"]


def run_whole(cfg: ModelConfig, prompts: torch.Tensor, steps: int, seed: int = 0):
    model = RefDecoder(cfg, init_weights(cfg, seed))
    return model.generate(prompts, steps)


def tiny_prompts(cfg: ModelConfig, batch: int = 2, length: int = 64, seed: int = 1) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (batch, length), generator=g)
