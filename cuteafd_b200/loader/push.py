"""Push loader: one coordinator reads every tensor of a snapshot once, in file order, and streams the pieces each
rank owns to that rank; the other ranks never open a weight file.

    plan   = build_plan(catalog, owners)          # coordinator: which rows of which tensor go to which ranks
    tensors = push_load(directory, owners, ...)   # every rank calls this; returns the tensors this rank owns

``owners(name, shape)`` returns, per tensor, a list of ``(rank, first_row, rows)`` windows (``rows`` -1 = to the
end; the same window may go to several ranks, and a tensor nobody owns is skipped without being read).  The plan
travels by ``broadcast_object_list``; the data by point-to-point sends with a small ring of requests in flight, so the
coordinator reads the next tensor while earlier ones are still on the wire.  A receiver may pass ``transform`` to
convert a piece as it lands (cast, device copy, load-time quantisation), so full-precision pieces never pile up.

On one NVSwitch box every rank could read the page cache itself (``load.load_gqa_engine_weights`` does); the push
form reads each byte from storage exactly once, which is what matters for a cold 600 GB checkpoint, and it is the
shape a multi-host deployment needs.  Process groups: gloo for CPU staging (tests), NCCL for device tensors.

Counterpart: rust/crates/cuteafd-loader/src/push_load.rs + push_load/ (coordinator reads shards once and pushes
slices through RDMA rings; device-side FP8 quantisation from ring slots, native/shared/cuda/fp8_load_quant.cu).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Callable

import torch
import torch.distributed as dist

from .safetensors_io import DTYPES, Catalog


@dataclass(frozen=True)
class PushItem:
    name: str
    dtype: str                  # safetensors dtype tag
    shape: tuple[int, ...]      # shape of the piece (first dimension = rows of the window)
    first_row: int
    rank: int


@dataclass
class PushStats:
    tensors_read: int = 0
    bytes_read: int = 0
    bytes_sent: int = 0
    bytes_kept: int = 0         # pieces the coordinator owns itself


Owners = Callable[[str, tuple[int, ...]], list[tuple[int, int, int]]]


def build_plan(cat: Catalog, owners: Owners) -> list[PushItem]:
    """Pieces in file order (tensors sorted by file and offset: the coordinator's reads are sequential)."""
    entries = sorted(cat.entries.values(), key=lambda e: (e.file, e.begin))
    plan: list[PushItem] = []
    for e in entries:
        for rank, first, rows in owners(e.name, e.shape) or ():
            total = e.shape[0] if e.shape else 1
            n = total - first if rows < 0 else rows
            if first < 0 or n <= 0 or first + n > total:
                raise ValueError(f"{e.name}: window [{first}, {first + n}) outside {total} rows")
            plan.append(PushItem(e.name, e.dtype, (n, *e.shape[1:]) if e.shape else (), first, rank))
    return plan


def _torch_dtype(tag: str) -> torch.dtype:
    return DTYPES[tag][0] if isinstance(DTYPES[tag], tuple) else DTYPES[tag]


def push_load(directory: str | None, owners: Owners | None, group=None, coordinator: int = 0, ring: int = 4,
              transform: Callable[[str, int, torch.Tensor], torch.Tensor] | None = None,
              device: torch.device | str = "cpu") -> tuple[dict[str, list[tuple[int, torch.Tensor]]], PushStats]:
    """Collective over ``group``.  Only the coordinator needs ``directory`` and ``owners``.  Returns
    ({tensor name: [(first_row, piece), ...]} for this rank, the coordinator's statistics).  ``device`` is where
    receive buffers live (NCCL groups need CUDA buffers)."""
    group = group or dist.group.WORLD
    rank = dist.get_rank(group)
    src = dist.get_global_rank(group, coordinator) if hasattr(dist, "get_global_rank") else coordinator
    box: list = [None]
    cat = None
    if rank == coordinator:
        cat = Catalog(directory)
        box[0] = build_plan(cat, owners)
    dist.broadcast_object_list(box, src=src, group=group)
    plan: list[PushItem] = box[0]
    mine: dict[str, list[tuple[int, torch.Tensor]]] = {}
    stats = PushStats()
    keep = transform or (lambda name, first, t: t)

    def viewable(t: torch.Tensor) -> torch.Tensor:
        # transports move bytes: 8-bit float tags travel as uint8
        return t.view(torch.uint8) if t.dtype in (torch.float8_e4m3fn, torch.float8_e5m2) else t

    if rank == coordinator:
        pending: list = []
        current, whole = None, None
        for it in plan:
            if it.name != current:
                current = it.name
                whole = cat.read(it.name)                     # one read per tensor, whatever the number of windows
                stats.tensors_read += 1
                stats.bytes_read += whole.numel() * whole.element_size()
            piece = whole[it.first_row: it.first_row + it.shape[0]] if whole.dim() else whole
            if it.rank == coordinator:
                mine.setdefault(it.name, []).append((it.first_row, keep(it.name, it.first_row, piece.clone().to(device))))
                stats.bytes_kept += piece.numel() * piece.element_size()
                continue
            buf = viewable(piece.contiguous()).to(device)
            pending.append((dist.isend(buf, dist.get_global_rank(group, it.rank) if hasattr(dist, "get_global_rank") else it.rank,
                                       group=group), buf))
            stats.bytes_sent += buf.numel() * buf.element_size()
            while len(pending) >= ring:
                pending.pop(0)[0].wait()
        for req, _ in pending:
            req.wait()
        cat.close()
    else:
        inflight: list = []

        def land(entry) -> None:
            req, it, buf = entry
            req.wait()
            t = buf.view(_torch_dtype(it.dtype)) if buf.dtype == torch.uint8 and _torch_dtype(it.dtype) != torch.uint8 else buf
            mine.setdefault(it.name, []).append((it.first_row, keep(it.name, it.first_row, t)))

        for it in plan:
            if it.rank != rank:
                continue
            dt = _torch_dtype(it.dtype)
            wire = torch.uint8 if dt in (torch.float8_e4m3fn, torch.float8_e5m2) else dt
            buf = torch.empty(it.shape, dtype=wire, device=device)
            inflight.append((dist.irecv(buf, src, group=group), it, buf))
            while len(inflight) >= ring:
                land(inflight.pop(0))
        for e in inflight:
            land(e)
    return mine, stats


def expert_parallel_owners(attention_ranks: list[int], expert_ranks: list[int], num_experts: int) -> Owners:
    """The usual AFD split: routed experts by contiguous id range over the expert ranks, everything else to every
    attention rank."""
    import re
    per = -(-num_experts // max(1, len(expert_ranks)))
    pat = re.compile(r"\.mlp\.experts\.(\d+)\.")

    def owners(name: str, shape: tuple[int, ...]) -> list[tuple[int, int, int]]:
        m = pat.search(name)
        if m:
            return [(expert_ranks[min(int(m.group(1)) // per, len(expert_ranks) - 1)], 0, -1)]
        return [(r, 0, -1) for r in attention_ranks]
    return owners
