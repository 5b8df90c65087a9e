"""Bounded asynchronous JSONL trace writer (one record per decode round) and NVTX ranges.

Records are queued and written by a background thread; when the queue is full records are
dropped and counted, never blocking the serve loop.  Counterpart:
rust/crates/cuteafd-daemon/src/shared/speculation_trace.rs:1-50.
"""
from __future__ import annotations

import contextlib
import json
import queue
import threading
import time


class JsonlTrace:
    def __init__(self, path: str, capacity: int = 4096):
        self.q: "queue.Queue[dict | None]" = queue.Queue(maxsize=capacity)
        self.dropped = 0
        self.f = open(path, "a", buffering=1)
        self.t = threading.Thread(target=self._run, daemon=True)
        self.t.start()

    def record(self, **fields) -> None:
        fields.setdefault("ts", time.time())
        try:
            self.q.put_nowait(fields)
        except queue.Full:
            self.dropped += 1

    def _run(self) -> None:
        while True:
            item = self.q.get()
            if item is None:
                break
            self.f.write(json.dumps(item) + "\n")

    def close(self) -> None:
        self.q.put(None)
        self.t.join(timeout=5)
        self.f.close()


@contextlib.contextmanager
def nvtx(name: str):
    try:
        import torch
        on = torch.cuda.is_available()
    except ImportError:
        on = False
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()
