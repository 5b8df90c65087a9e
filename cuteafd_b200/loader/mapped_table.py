"""Host-RAM lookup tables that are too large (or too cold) for GPU memory: a row-addressable table memory-mapped
from its checkpoint file, gathered by a small thread pool, with lookahead prefetch of the rows the next steps will
need and hit / miss statistics.

Use: per-token embedding-like tables consulted once per token (DeepSeek "engram" / per-layer-embedding tables in the
reference, rust/crates/cuteafd-loader/src/formats/mapped_table.rs, which gathers with io_uring pools).  Here the
gather is a chunked fancy-index over ``numpy.memmap`` executed on worker threads (page-cache reads release the
GIL), into pinned staging buffers that are copied to the device on the caller's stream.
"""
from __future__ import annotations

import threading
from concurrent.futures import Future, ThreadPoolExecutor
from dataclasses import dataclass, field

import numpy as np
import torch


@dataclass
class TableStats:
    gathers: int = 0
    rows: int = 0
    prefetched_rows: int = 0
    prefetch_hits: int = 0
    bytes_read: int = 0


class MappedTable:
    def __init__(self, path: str, rows: int, width: int, dtype=np.float16, offset: int = 0, workers: int = 4,
                 chunk_rows: int = 256, cache_rows: int = 65536):
        self.rows, self.width, self.dtype = rows, width, np.dtype(dtype)
        self.mm = np.memmap(path, dtype=self.dtype, mode="r", offset=offset, shape=(rows, width))
        self.pool = ThreadPoolExecutor(max_workers=workers, thread_name_prefix="mapped-table")
        self.chunk_rows = chunk_rows
        self.stats = TableStats()
        self._cache: dict[int, np.ndarray] = {}          # prefetched rows by id (bounded FIFO)
        self._order: list[int] = []
        self._cache_rows = cache_rows
        self._lock = threading.Lock()
        self._pending: list[Future] = []

    @staticmethod
    def from_safetensors(catalog, name: str, **kw) -> "MappedTable":
        """Map a 2-D tensor of a safetensors file in place (no copy)."""
        e = catalog.entries[name]
        np_dtype = {"F16": np.float16, "BF16": np.uint16, "F32": np.float32, "U8": np.uint8, "I8": np.int8}[e.dtype]
        return MappedTable(e.file, e.shape[0], e.shape[1], np_dtype, offset=e.begin, **kw)

    # ---- prefetch ---------------------------------------------------------------------------------------------
    def prefetch(self, ids) -> None:
        """Start reading rows that a later ``gather`` will ask for (lookahead: the next tokens of a prompt, the
        drafts of a speculative step)."""
        ids = np.unique(np.asarray(ids, dtype=np.int64))
        with self._lock:
            ids = ids[[int(i) not in self._cache for i in ids]] if len(ids) else ids
        for c in range(0, len(ids), self.chunk_rows):
            part = ids[c:c + self.chunk_rows]
            self._pending.append(self.pool.submit(self._load, part))

    def _load(self, ids: np.ndarray) -> None:
        data = np.ascontiguousarray(self.mm[ids])
        with self._lock:
            for i, row in zip(ids.tolist(), data):
                if i not in self._cache:
                    self._cache[i] = row
                    self._order.append(i)
            while len(self._order) > self._cache_rows:
                self._cache.pop(self._order.pop(0), None)
            self.stats.prefetched_rows += len(ids)
            self.stats.bytes_read += data.nbytes

    def drain(self) -> None:
        for f in self._pending:
            f.result()
        self._pending.clear()

    # ---- gather -----------------------------------------------------------------------------------------------
    def gather(self, ids, out: torch.Tensor | None = None) -> torch.Tensor:
        """Rows ``ids`` as a [n, width] tensor (pinned when CUDA is present so the device copy can be async)."""
        ids = np.asarray(ids, dtype=np.int64)
        n = len(ids)
        if out is None:
            out = torch.empty(n, self.width, dtype=_torch_dtype(self.dtype))
            if torch.cuda.is_available():
                out = out.pin_memory()
        dst = out.numpy() if out.dtype != torch.bfloat16 else out.view(torch.int16).numpy().view(np.uint16)
        self.drain()
        miss_pos, miss_ids = [], []
        with self._lock:
            for p, i in enumerate(ids.tolist()):
                row = self._cache.get(i)
                if row is not None:
                    dst[p] = row
                    self.stats.prefetch_hits += 1
                else:
                    miss_pos.append(p); miss_ids.append(i)
        if miss_ids:
            mp, mi = np.asarray(miss_pos), np.asarray(miss_ids)
            futs = [self.pool.submit(lambda a, b: dst.__setitem__(a, self.mm[b]), mp[c:c + self.chunk_rows], mi[c:c + self.chunk_rows])
                    for c in range(0, len(mi), self.chunk_rows)]
            for f in futs:
                f.result()
            self.stats.bytes_read += len(mi) * self.width * self.dtype.itemsize
        self.stats.gathers += 1
        self.stats.rows += n
        return out

    def close(self) -> None:
        self.pool.shutdown(wait=True)


def _torch_dtype(dt: np.dtype) -> torch.dtype:
    return {np.dtype(np.float16): torch.float16, np.dtype(np.float32): torch.float32, np.dtype(np.uint16): torch.bfloat16,
            np.dtype(np.uint8): torch.uint8, np.dtype(np.int8): torch.int8}[dt]
