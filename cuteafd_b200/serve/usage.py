"""Request accounting in sqlite: one accounting row per finished request (kept), and a full request log — the request
body and the reply text — that is pruned to the last 24 hours.

    log = UsageLog("usage.sqlite")
    log.record(model, api, usage, seconds, finish, request=body, reply=text, ttft=0.21, client="10.0.0.7")
    log.summary(24)          # totals, by API flavour, draft acceptance, cached-token share
    log.hourly(24)           # one bucket per hour: requests, tokens, busy seconds
    log.requests(limit=50)   # newest first, without bodies
    log.request(rowid)       # one entry with its body and reply (while the 24 h log still has it)

HTTP: ``/console/usage/summary``, ``/console/usage/hourly``, ``/console/usage/requests?limit=N``,
``/console/usage/request/<id>``.  Writes happen on the serving threads under a lock; sqlite runs in WAL mode so the
``cuteafd usage`` command can read the file while the server writes it.

Counterpart: rust/crates/cuteafd-usage/src/{store.rs,query.rs,log/*,http.rs:53-66}.
"""
from __future__ import annotations

import json
import sqlite3
import threading
import time

LOG_SECONDS = 24 * 3600
BODY_LIMIT = 256 << 10                   # bytes of request / reply kept per entry


class UsageLog:
    def __init__(self, path: str = ":memory:", clock=time.time):
        self.db = sqlite3.connect(path, check_same_thread=False)
        self.lock = threading.Lock()
        self.clock = clock
        self._since_prune = 0
        if path != ":memory:":
            try:
                self.db.execute("PRAGMA journal_mode=WAL")
            except sqlite3.DatabaseError:
                pass
        self.db.execute("CREATE TABLE IF NOT EXISTS requests (id INTEGER PRIMARY KEY AUTOINCREMENT, ts REAL, model TEXT, "
                        "api TEXT, prompt_tokens INT, completion_tokens INT, cached_tokens INT, proposed INT, accepted INT, "
                        "seconds REAL, finish TEXT, ttft REAL, client TEXT, detail TEXT)")
        have = {r[1] for r in self.db.execute("PRAGMA table_info(requests)")}
        for col, typ in (("ttft", "REAL"), ("client", "TEXT"), ("detail", "TEXT")):     # files written before these existed
            if col not in have:
                self.db.execute(f"ALTER TABLE requests ADD COLUMN {col} {typ}")
        self.db.execute("CREATE TABLE IF NOT EXISTS request_log (id INTEGER PRIMARY KEY, ts REAL, request TEXT, reply TEXT)")
        self.db.execute("CREATE INDEX IF NOT EXISTS requests_ts ON requests (ts)")
        self.db.execute("CREATE INDEX IF NOT EXISTS request_log_ts ON request_log (ts)")
        self.db.commit()

    # ---- writing --------------------------------------------------------------------------
    def record(self, model: str, api: str, usage: dict, seconds: float, finish: str, request=None, reply: str | None = None,
               ttft: float | None = None, client: str = "") -> int:
        sp = usage.get("speculation", {})
        now = self.clock()
        with self.lock:
            cur = self.db.execute(
                "INSERT INTO requests (ts, model, api, prompt_tokens, completion_tokens, cached_tokens, proposed, accepted, "
                "seconds, finish, ttft, client, detail) VALUES (?,?,?,?,?,?,?,?,?,?,?,?,?)",
                (now, model, api, usage.get("prompt_tokens", 0), usage.get("completion_tokens", 0),
                 usage.get("cached_tokens", 0), sp.get("proposed", 0), sp.get("accepted", 0), seconds, finish, ttft, client,
                 usage.get("finish_detail", "")))
            rid = cur.lastrowid
            if request is not None or reply is not None:
                body = request if isinstance(request, str) else json.dumps(request, default=str)
                self.db.execute("INSERT INTO request_log VALUES (?,?,?,?)",
                                (rid, now, (body or "")[:BODY_LIMIT], (reply or "")[:BODY_LIMIT]))
            self._since_prune += 1
            if self._since_prune >= 64:
                self._prune(now)
            self.db.commit()
        return rid

    def _prune(self, now: float) -> None:
        self.db.execute("DELETE FROM request_log WHERE ts < ?", (now - LOG_SECONDS,))
        self._since_prune = 0

    def prune(self) -> None:
        with self.lock:
            self._prune(self.clock())
            self.db.commit()

    # ---- queries --------------------------------------------------------------------------
    def summary(self, hours: float = 24.0) -> dict:
        since = self.clock() - hours * 3600
        with self.lock:
            row = self.db.execute("SELECT COUNT(*), COALESCE(SUM(prompt_tokens),0), COALESCE(SUM(completion_tokens),0), "
                                  "COALESCE(SUM(cached_tokens),0), COALESCE(SUM(proposed),0), COALESCE(SUM(accepted),0), "
                                  "COALESCE(SUM(seconds),0), AVG(ttft) FROM requests WHERE ts >= ?", (since,)).fetchone()
            per = self.db.execute("SELECT api, COUNT(*) FROM requests WHERE ts >= ? GROUP BY api", (since,)).fetchall()
            fin = self.db.execute("SELECT finish, COUNT(*) FROM requests WHERE ts >= ? GROUP BY finish", (since,)).fetchall()
            loops = self.db.execute("SELECT COUNT(*) FROM requests WHERE ts >= ? AND detail = 'repetition'", (since,)).fetchone()[0]
        n, p, c, cached, prop, acc, sec, ttft = row
        return {"hours": hours, "requests": n, "prompt_tokens": p, "completion_tokens": c, "cached_tokens": cached,
                "cached_share": (cached / p) if p else None, "draft_acceptance": (acc / prop) if prop else None,
                "busy_seconds": sec, "mean_ttft_s": ttft, "by_api": dict(per), "by_finish": dict(fin), "loop_aborts": loops}

    def hourly(self, hours: int = 24) -> list[dict]:
        now = self.clock()
        since = now - hours * 3600
        with self.lock:
            rows = self.db.execute("SELECT CAST((ts - ?) / 3600 AS INT) AS h, COUNT(*), SUM(prompt_tokens), SUM(completion_tokens), "
                                   "SUM(seconds) FROM requests WHERE ts >= ? GROUP BY h ORDER BY h", (since, since)).fetchall()
        got = {h: (n, p, c, s) for h, n, p, c, s in rows}
        return [{"hour_start": since + h * 3600, "requests": got.get(h, (0, 0, 0, 0))[0], "prompt_tokens": got.get(h, (0, 0, 0, 0))[1] or 0,
                 "completion_tokens": got.get(h, (0, 0, 0, 0))[2] or 0, "busy_seconds": got.get(h, (0, 0, 0, 0))[3] or 0.0}
                for h in range(int(hours))]

    _COLS = ("id", "ts", "model", "api", "prompt_tokens", "completion_tokens", "cached_tokens", "proposed", "accepted", "seconds",
             "finish", "ttft", "client", "detail")

    def requests(self, limit: int = 50, before_id: int | None = None) -> list[dict]:
        q = f"SELECT {', '.join(self._COLS)} FROM requests"
        args: tuple = ()
        if before_id is not None:
            q, args = q + " WHERE id < ?", (before_id,)
        with self.lock:
            rows = self.db.execute(q + " ORDER BY id DESC LIMIT ?", args + (max(1, min(int(limit), 1000)),)).fetchall()
        return [dict(zip(self._COLS, r)) for r in rows]

    def request(self, rid: int) -> dict | None:
        with self.lock:
            row = self.db.execute(f"SELECT {', '.join(self._COLS)} FROM requests WHERE id = ?", (rid,)).fetchone()
            if row is None:
                return None
            body = self.db.execute("SELECT request, reply FROM request_log WHERE id = ?", (rid,)).fetchone()
        out = dict(zip(self._COLS, row))
        out["logged"] = body is not None
        if body is not None:
            out["request"], out["reply"] = body
        return out


def usage_report(path: str, hours: float) -> dict:
    log = UsageLog(path)
    return {"summary": log.summary(hours), "hourly": log.hourly(int(max(1, min(hours, 168))))}
