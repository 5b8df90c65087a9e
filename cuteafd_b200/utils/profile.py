"""``PROFILE=mode[,mode...]`` for one launch of ``cuteafd serve``: cheap, host-side instrumentation that is off unless
asked for.

* ``draft-timing``   wraps the drafter's ``draft`` / ``accept`` / ``begin``: calls and seconds per call kind, and the
                     share of the decode loop they take (shown under ``profile`` in ``/v1/stats``).
* ``expert-routes``  appends the backend's expert usage (routed tokens per layer and expert, imbalance) to
                     ``<dir>/expert_routes.jsonl`` every ``period`` decode rounds.
* ``census``         appends the decode graph bank's inventory (captured geometries, replays, eager steps) and the
                     scheduler's verify-row histogram to ``<dir>/census.jsonl`` every ``period`` rounds.
* ``step-timing``    wall time of every scheduler step by kind (prefill / decode / idle) as running totals.
* ``transport-timing`` / ``expert-timing``  for expert workers reached over TCP (``serve --expert-workers``): per worker,
                     the round trip, the worker's own compute time from its reply header, and their difference
                     (``transport``); ``expert-timing`` adds the slowest worker's share over the mean (imbalance).
                     Both read what the links already record.

The modes only read counters the serve loop already keeps, or time host calls; none adds a device synchronisation.
Device-side profiles (``ncu``) are taken on small standalone cases of a kernel, never by wrapping a server.

Counterpart: ``PROFILE=census,transport-timing,expert-timing,expert-routes,draft-timing`` of the reference's launcher
(docs/options.md:944-955).
"""
from __future__ import annotations

import json
import os
import time

MODES = ("draft-timing", "expert-routes", "census", "step-timing", "transport-timing", "expert-timing")


def parse_modes(text: str) -> list[str]:
    modes = [m.strip() for m in (text or "").split(",") if m.strip()]
    bad = [m for m in modes if m not in MODES]
    if bad:
        raise ValueError(f"unknown PROFILE mode {bad[0]!r} (choose from {', '.join(MODES)})")
    return modes


class _Timed:
    def __init__(self, inner, book: dict):
        self._inner, self._book = inner, book

    def __getattr__(self, name):
        v = getattr(self._inner, name)
        if name not in ("draft", "accept", "begin", "offer") or not callable(v):
            return v

        def timed(*a, **k):
            t0 = time.perf_counter()
            try:
                return v(*a, **k)
            finally:
                rec = self._book.setdefault(name, [0, 0.0])
                rec[0] += 1
                rec[1] += time.perf_counter() - t0
        return timed


class Profile:
    def __init__(self, modes: list[str], out_dir: str = ".", period: int = 64):
        self.modes, self.dir, self.period = modes, out_dir, max(1, period)
        self.draft: dict[str, list] = {}
        self.steps = {"prefill": [0, 0.0], "decode": [0, 0.0], "idle": [0, 0.0]}
        self._last_round = 0
        if any(m in modes for m in ("expert-routes", "census")):
            os.makedirs(out_dir, exist_ok=True)

    def attach(self, sched) -> "Profile":
        if "draft-timing" in self.modes:
            sched.drafter = _Timed(sched.drafter, self.draft)
        if any(m in self.modes for m in ("expert-routes", "census", "step-timing")):
            inner = sched.step

            def step():
                before = (sched.stats.prefill_tokens, sched.stats.decode_rounds)
                t0 = time.perf_counter()
                did = inner()
                dt = time.perf_counter() - t0
                kind = "decode" if sched.stats.decode_rounds != before[1] else "prefill" if sched.stats.prefill_tokens != before[0] else "idle"
                self.steps[kind][0] += 1
                self.steps[kind][1] += dt
                if sched.stats.decode_rounds - self._last_round >= self.period:
                    self._last_round = sched.stats.decode_rounds
                    self.flush(sched)
                return did
            sched.step = step
        sched.profile = self
        self.remote = getattr(sched.be, "remote_experts", None)      # TCP expert workers, when the backend uses them
        return self

    def flush(self, sched) -> None:
        now = time.time()
        if "expert-routes" in self.modes and hasattr(sched.be, "expert_usage"):
            self._append("expert_routes.jsonl", {"ts": now, "round": sched.stats.decode_rounds, "usage": sched.be.expert_usage()})
        if "census" in self.modes:
            rec = {"ts": now, "round": sched.stats.decode_rounds, "verify_row_hist": dict(sched.stats.verify_row_hist)}
            if hasattr(sched.be, "graph_stats"):
                rec["graphs"] = sched.be.graph_stats()
            self._append("census.jsonl", rec)

    def _append(self, name: str, rec: dict) -> None:
        with open(os.path.join(self.dir, name), "a") as f:
            f.write(json.dumps(rec) + "\n")

    def report(self) -> dict:
        out: dict = {"modes": self.modes}
        if "draft-timing" in self.modes:
            out["draft"] = {k: {"calls": c, "seconds": round(s, 6), "mean_us": round(s / c * 1e6, 2) if c else None}
                            for k, (c, s) in sorted(self.draft.items())}
            dec = self.steps["decode"][1]
            if dec:
                out["draft"]["share_of_decode"] = round(sum(s for _, s in self.draft.values()) / dec, 4)
        remote = getattr(self, "remote", None)
        if remote is not None and ("transport-timing" in self.modes or "expert-timing" in self.modes):
            rows = remote.timing()
            if "transport-timing" in self.modes:
                out["transport"] = [{k: r[k] for k in ("experts", "ok", "calls", "sent_bytes", "recv_bytes", "round_trip", "transport")} for r in rows]
            if "expert-timing" in self.modes:
                means = [r["compute"]["mean_us"] for r in rows if r["compute"]]
                out["experts"] = {"workers": [{k: r[k] for k in ("experts", "calls", "compute")} for r in rows],
                                  "imbalance": round(max(means) / (sum(means) / len(means)), 3) if means and sum(means) else None}
        if "step-timing" in self.modes or "draft-timing" in self.modes:
            out["steps"] = {k: {"count": c, "seconds": round(s, 6)} for k, (c, s) in self.steps.items()}
        return out
