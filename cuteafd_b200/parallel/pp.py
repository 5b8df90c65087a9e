"""Pipeline-stage hop: the residual stream of a step moves from the GPU that owns layers [0, k) to the GPU that
owns layers [k, L) with NCCL point-to-point calls issued on a side stream, so the sender's next micro-step and
the receiver's previous one keep computing.

This is the one path that stays on NCCL by design (a hop is a plain contiguous copy with nothing to fuse into).
The reference moves residual rows between its two coordinator GPUs the same way at four possible points
(Entry / BeforeLayer / AfterAttention / Exit; rust/crates/cuteafd-loader/src/placement/residual.rs:62-71 and
rust/crates/cuteafd-daemon/src/shared/peer_split/hop.rs).
"""
from __future__ import annotations

from dataclasses import dataclass

import torch
import torch.distributed as dist


@dataclass
class StagePlan:
    """Layer ranges of the pipeline stages: stage s owns layers [bounds[s], bounds[s+1])."""
    bounds: list[int]

    @staticmethod
    def even(num_layers: int, stages: int) -> "StagePlan":
        return StagePlan([round(i * num_layers / stages) for i in range(stages + 1)])

    def stage_of(self, layer: int) -> int:
        for s in range(len(self.bounds) - 1):
            if self.bounds[s] <= layer < self.bounds[s + 1]:
                return s
        raise IndexError(layer)

    def layers(self, stage: int) -> range:
        return range(self.bounds[stage], self.bounds[stage + 1])


class Hop:
    """One direction of a stage boundary.  ``send`` / ``recv`` enqueue the transfer on a side stream after the
    producing work (``send``) and make the consuming stream wait for it (``recv``); with ``backend="gloo"`` (CPU
    tests) the calls are plain blocking send / recv."""

    def __init__(self, peer: int, group=None, device: torch.device | None = None):
        self.peer, self.group = peer, group
        self.cuda = device is not None and device.type == "cuda"
        self.stream = torch.cuda.Stream(device=device) if self.cuda else None
        self.bytes_moved = 0

    def send(self, rows: torch.Tensor) -> None:
        self.bytes_moved += rows.numel() * rows.element_size()
        if not self.cuda:
            dist.send(rows.contiguous(), self.peer, group=self.group)
            return
        self.stream.wait_stream(torch.cuda.current_stream())       # after the kernels that produced the rows
        with torch.cuda.stream(self.stream):
            dist.send(rows, self.peer, group=self.group)
        rows.record_stream(self.stream)

    def recv(self, out: torch.Tensor) -> torch.Tensor:
        self.bytes_moved += out.numel() * out.element_size()
        if not self.cuda:
            dist.recv(out, self.peer, group=self.group)
            return out
        self.stream.wait_stream(torch.cuda.current_stream())       # the buffer's previous readers are done
        with torch.cuda.stream(self.stream):
            dist.recv(out, self.peer, group=self.group)
        torch.cuda.current_stream().wait_stream(self.stream)       # consumers start after the rows have landed
        return out


class RingHop(Hop):
    """A hop with its own staging ring, so that transfers overlap the compute on both sides: ``send`` copies the rows
    into a ring slot (the caller may overwrite its buffer right away) and sends from there on the side stream;
    ``recv`` lands in a ring slot on the side stream (it can be in flight while the consumer still works on the
    previous micro-batch) and the consumer copies out.  A slot is reused only after its previous transfer / copy-out
    has finished (events)."""

    def __init__(self, peer: int, group=None, device: torch.device | None = None, rows: int = 0, width: int = 0,
                 dtype: torch.dtype = torch.bfloat16, slots: int = 2):
        super().__init__(peer, group, device)
        self.ring = [torch.empty(rows, width, dtype=dtype, device=device) for _ in range(slots)] if self.cuda else []
        self.free_ev: list = [None] * slots
        self.k = 0

    def send(self, rows: torch.Tensor) -> None:
        if not self.cuda:
            return super().send(rows)
        self.bytes_moved += rows.numel() * rows.element_size()
        k, self.k = self.k, (self.k + 1) % len(self.ring)
        cur = torch.cuda.current_stream()
        if self.free_ev[k] is not None:
            cur.wait_event(self.free_ev[k])                          # the slot's previous send has left
        buf = self.ring[k][:rows.shape[0]]
        buf.copy_(rows)
        self.stream.wait_stream(cur)
        with torch.cuda.stream(self.stream):
            dist.send(buf, self.peer, group=self.group)
            ev = torch.cuda.Event()
            ev.record(self.stream)
        self.free_ev[k] = ev

    def recv(self, out: torch.Tensor) -> torch.Tensor:
        if not self.cuda:
            return super().recv(out)
        self.bytes_moved += out.numel() * out.element_size()
        k, self.k = self.k, (self.k + 1) % len(self.ring)
        if self.free_ev[k] is not None:
            self.stream.wait_event(self.free_ev[k])                  # the slot's previous rows were copied out
        buf = self.ring[k][:out.shape[0]]
        with torch.cuda.stream(self.stream):
            dist.recv(buf, self.peer, group=self.group)
        cur = torch.cuda.current_stream()
        cur.wait_stream(self.stream)
        out.copy_(buf)
        ev = torch.cuda.Event()
        ev.record(cur)
        self.free_ev[k] = ev
        return out


def run_pipelined(stage: int, stages: int, micro_batches: list[torch.Tensor], stage_fn, hop_prev: Hop | None,
                  hop_next: Hop | None, out_like) -> list[torch.Tensor]:
    """Drive one stage over a list of micro-batches: receive (unless first stage), compute, send (unless last).
    Micro-batch m+1's receive is posted before micro-batch m's compute finishes, so hops overlap compute."""
    outs = []
    for mb in micro_batches:
        x = mb if stage == 0 else hop_prev.recv(out_like(mb))
        y = stage_fn(x)
        if stage < stages - 1:
            hop_next.send(y)
        outs.append(y)
    return outs
