"""Embedding cache: tower outputs keyed by the content hash of the media bytes, bounded in bytes, least recently used
entry out first.  A repeated image (a conversation that re-sends its history) costs one dictionary lookup instead of a
tower pass.  Counterpart: the embedding cache of rust/crates/cuteafd-engine/src/media/."""
from __future__ import annotations

import threading
from collections import OrderedDict

import torch


class EmbeddingCache:
    def __init__(self, max_bytes: int = 1 << 30):
        self.max_bytes = max_bytes
        self.bytes = 0
        self.hits = self.misses = self.evictions = 0
        self._d: "OrderedDict[bytes, torch.Tensor]" = OrderedDict()
        self._lock = threading.Lock()

    def get(self, key: bytes) -> torch.Tensor | None:
        with self._lock:
            t = self._d.get(key)
            if t is None:
                self.misses += 1
                return None
            self._d.move_to_end(key)
            self.hits += 1
            return t

    def put(self, key: bytes, value: torch.Tensor) -> None:
        size = value.numel() * value.element_size()
        if size > self.max_bytes:
            return
        with self._lock:
            old = self._d.pop(key, None)
            if old is not None:
                self.bytes -= old.numel() * old.element_size()
            self._d[key] = value
            self.bytes += size
            while self.bytes > self.max_bytes:
                _, v = self._d.popitem(last=False)
                self.bytes -= v.numel() * v.element_size()
                self.evictions += 1

    def describe(self) -> dict:
        return {"entries": len(self._d), "bytes": self.bytes, "hits": self.hits, "misses": self.misses,
                "evictions": self.evictions}
