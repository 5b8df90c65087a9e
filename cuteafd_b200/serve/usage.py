"""Request accounting in sqlite: one row per finished request, 24-hour summaries.

Counterpart: rust/crates/cuteafd-usage/src/{store.rs,query.rs,http.rs:53-66}.
"""
from __future__ import annotations

import sqlite3
import threading
import time


class UsageLog:
    def __init__(self, path: str = ":memory:"):
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.lock = threading.Lock()
        self.db.execute("CREATE TABLE IF NOT EXISTS requests (ts REAL, model TEXT, api TEXT, prompt_tokens INT, "
                        "completion_tokens INT, cached_tokens INT, proposed INT, accepted INT, seconds REAL, finish TEXT)")
        self.db.commit()

    def record(self, model: str, api: str, usage: dict, seconds: float, finish: str) -> None:
        sp = usage.get("speculation", {})
        with self.lock:
            self.db.execute("INSERT INTO requests VALUES (?,?,?,?,?,?,?,?,?,?)",
                            (time.time(), model, api, usage.get("prompt_tokens", 0), usage.get("completion_tokens", 0),
                             usage.get("cached_tokens", 0), sp.get("proposed", 0), sp.get("accepted", 0), seconds, finish))
            self.db.commit()

    def summary(self, hours: float = 24.0) -> dict:
        since = time.time() - hours * 3600
        with self.lock:
            row = self.db.execute("SELECT COUNT(*), COALESCE(SUM(prompt_tokens),0), COALESCE(SUM(completion_tokens),0), "
                                  "COALESCE(SUM(cached_tokens),0), COALESCE(SUM(proposed),0), COALESCE(SUM(accepted),0), "
                                  "COALESCE(SUM(seconds),0) FROM requests WHERE ts >= ?", (since,)).fetchone()
            per = self.db.execute("SELECT api, COUNT(*) FROM requests WHERE ts >= ? GROUP BY api", (since,)).fetchall()
        n, p, c, cached, prop, acc, sec = row
        return {"hours": hours, "requests": n, "prompt_tokens": p, "completion_tokens": c, "cached_tokens": cached,
                "draft_acceptance": (acc / prop) if prop else None, "busy_seconds": sec, "by_api": dict(per)}


def usage_report(path: str, hours: float) -> dict:
    return UsageLog(path).summary(hours)
