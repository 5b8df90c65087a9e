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


def prewarm_from_trace(path: str, top: int = 32) -> dict:
    """A decode-graph prewarm list from a speculation trace: every round's step geometry (sequences, rows, longest run
    = 1 + the most drafts one request kept) counted, the ``top`` most frequent first.  The result has the shape
    ``serve --prewarm FILE`` reads, so the traffic of one run warms the graphs of the next without holding the server
    that produced it.

    Counterpart: scripts/dev/graph-prewarm-from-trace.py over ``GRAPH_TRACE`` snapshots (docs/shared-engine.md:719-741)."""
    import json
    seen: dict[tuple[int, int, int], int] = {}
    rounds = 0
    with open(path) as f:
        for line in f:
            line = line.strip()
            if not line:
                continue
            try:
                r = json.loads(line)
            except json.JSONDecodeError:
                continue                                     # a line cut short when the process ended
            if "requests" not in r or "rows" not in r:
                continue
            key = (len(r["requests"]), int(r["rows"]), 1 + max([int(k) for k in r.get("kept") or [0]] + [0]))
            if key[0] < 1 or key[1] < key[0]:
                continue
            seen[key] = seen.get(key, 0) + 1
            rounds += 1
    order = sorted(seen.items(), key=lambda kv: (-kv[1], kv[0]))
    return {"geometries": [list(k) for k, _ in order[:max(0, top)]], "seen": {",".join(map(str, k)): v for k, v in order},
            "rounds": rounds, "source": "speculation-trace"}

