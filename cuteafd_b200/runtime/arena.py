"""Weight arena: one planned allocation per device for a whole weight set, with aligned views into it.

    arena = WeightArena("cuda:0")
    arena.reserve("layers.0.wqkv", (q + 2 * kv, hidden), torch.bfloat16)      # pass 1: sizes only
    ...
    arena.allocate()                                                         # one buffer, tagged in the memory ledger
    arena.fill_rows("layers.0.wqkv", 0, q_rows)                               # pass 2: pieces land in place
    w = arena.view("layers.0.wqkv")

Why not one ``torch.empty`` per tensor: a 600 GB model has ~50 000 tensors; the caching allocator rounds each to its
block size and fragments, the peak while stacking experts doubles a layer's footprint, and nothing can say afterwards
where the memory went.  With the arena the size is known before a byte is read (so a model that does not fit fails
before loading, with the ledger's numbers), pieces are copied straight to their final place, and views start on 256-byte
boundaries (a multiple of the 16 bytes a tensor map's base address needs, and of the 128-byte L2 line).

Counterpart: rust/crates/cuteafd-daemon/src/shared/memory/weight_arena.rs (one preplanned allocation per device per
weight set with aligned views), weight_views.rs.
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import torch

from ..utils.memory_ledger import LEDGER, MemoryLedger

ALIGN = 256


@dataclass
class Slot:
    name: str
    shape: tuple[int, ...]
    dtype: torch.dtype
    offset: int
    nbytes: int


class ArenaError(RuntimeError):
    pass


class WeightArena:
    def __init__(self, device: str | torch.device = "cpu", owner: str = "weights", ledger: MemoryLedger | None = None):
        self.device = torch.device(device)
        self.owner = owner
        self.ledger = LEDGER if ledger is None else ledger
        self.slots: dict[str, Slot] = {}
        self.size = 0
        self.buf: torch.Tensor | None = None
        self.filled: dict[str, int] = {}            # rows written per slot (load completeness check)

    # ---- pass 1 ---------------------------------------------------------------------------
    def reserve(self, name: str, shape, dtype: torch.dtype) -> Slot:
        if self.buf is not None:
            raise ArenaError("the arena is already allocated")
        if name in self.slots:
            raise ArenaError(f"{name} reserved twice")
        shape = tuple(int(s) for s in shape)
        nbytes = math.prod(shape) * torch.empty((), dtype=dtype).element_size()
        slot = Slot(name, shape, dtype, self.size, nbytes)
        self.slots[name] = slot
        self.size += (nbytes + ALIGN - 1) // ALIGN * ALIGN
        return slot

    def check_fits(self, free_bytes: int, reserve_bytes: int = 0) -> None:
        """Refuse before loading when the plan cannot fit (``reserve_bytes``: what must stay free for KV, graphs...)."""
        if self.size + reserve_bytes > free_bytes:
            top = sorted(self.slots.values(), key=lambda s: -s.nbytes)[:5]
            raise ArenaError(
                f"{self.owner}: {self.size / 2**30:.2f} GiB of weights + {reserve_bytes / 2**30:.2f} GiB reserve do not fit "
                f"in {free_bytes / 2**30:.2f} GiB free on {self.device}; largest: "
                + ", ".join(f"{s.name} {s.nbytes / 2**20:.0f} MiB" for s in top))

    # ---- allocation -----------------------------------------------------------------------
    def allocate(self) -> "WeightArena":
        if self.buf is not None:
            return self
        with self.ledger.guard(f"weight arena {self.owner} ({self.size} bytes)"):
            # over-allocate by one alignment unit so that the first view can be moved onto a boundary
            raw = torch.empty(self.size + ALIGN, dtype=torch.uint8, device=self.device)
        shift = (-raw.data_ptr()) % ALIGN
        self.buf = raw[shift:shift + self.size]
        self._raw = raw
        self.ledger.tag_tensor("weights", self.owner, raw)        # views of it are then never counted again
        return self

    def view(self, name: str) -> torch.Tensor:
        if self.buf is None:
            raise ArenaError("allocate() first")
        s = self.slots[name]
        return self.buf[s.offset:s.offset + s.nbytes].view(s.dtype).view(s.shape)

    # ---- pass 2 ---------------------------------------------------------------------------
    def fill(self, name: str, src: torch.Tensor) -> torch.Tensor:
        v = self.view(name)
        if tuple(src.shape) != tuple(v.shape):
            raise ArenaError(f"{name}: got shape {tuple(src.shape)}, planned {tuple(v.shape)}")
        v.copy_(src, non_blocking=True)
        self.filled[name] = v.shape[0] if v.dim() else 1
        return v

    def fill_rows(self, name: str, first: int, src: torch.Tensor) -> None:
        """Write ``src`` at rows [first, first + len(src)) of the slot's leading dimension."""
        v = self.view(name)
        n = src.shape[0]
        if first < 0 or first + n > v.shape[0] or tuple(src.shape[1:]) != tuple(v.shape[1:]):
            raise ArenaError(f"{name}: rows [{first}, {first + n}) of shape {tuple(src.shape)} do not fit {tuple(v.shape)}")
        v[first:first + n].copy_(src, non_blocking=True)
        self.filled[name] = self.filled.get(name, 0) + n

    def missing(self) -> list[str]:
        """Slots that were not (completely) written."""
        out = []
        for n, s in self.slots.items():
            want = s.shape[0] if s.shape else 1
            if self.filled.get(n, 0) < want:
                out.append(n)
        return out

    def describe(self) -> dict:
        return {"device": str(self.device), "owner": self.owner, "bytes": self.size, "tensors": len(self.slots),
                "padding": self.size - sum(s.nbytes for s in self.slots.values()), "allocated": self.buf is not None}

    def release(self) -> None:
        self.buf = None
        self._raw = None
        self.ledger.release("weights", self.owner, str(self.device))
