"""``GET /metrics``: the scheduler's counters, the memory ledger and the GPU telemetry in the Prometheus text format.

Counters are the lifetime totals the scheduler keeps (they only grow); gauges are read at scrape time.  Nothing is
sampled for the scrape that the console does not already read, so scraping every few seconds costs nothing on the
serve loop.  The reference publishes the same numbers as JSON (``/v1/stats``, ``/v1/thermal``, ``/memory``); a
Prometheus view is what a fleet's monitoring stack expects.
"""
from __future__ import annotations

import time

_COUNTERS = {
    "admitted": "requests admitted", "finished": "requests finished", "failed": "requests failed by a worker error",
    "rejected": "requests refused for capacity (HTTP 429)", "prefill_tokens": "prompt tokens computed",
    "cached_tokens": "prompt tokens served from the prefix cache", "decode_rounds": "decode steps",
    "emitted_tokens": "tokens generated", "verify_rows": "rows verified (selected token + drafts)",
    "stalls": "decode rounds a request sat out waiting for KV pages", "quarantined": "sequences whose pages were quarantined",
    "loop_aborts": "replies ended by the repetition detector", "packed_steps": "prefill steps shared by several prompts",
}


def _line(name: str, value, labels: dict | None = None) -> str:
    lab = "{" + ",".join(f'{k}="{v}"' for k, v in sorted((labels or {}).items())) + "}" if labels else ""
    return f"cuteafd_{name}{lab} {value}"


def render(state) -> str:
    snap = state.sched.snapshot()
    out: list[str] = []

    def family(name: str, kind: str, help_: str, rows: list[str]) -> None:
        out.append(f"# HELP cuteafd_{name} {help_}")
        out.append(f"# TYPE cuteafd_{name} {kind}")
        out.extend(rows)
    for key, help_ in _COUNTERS.items():
        family(f"{key}_total", "counter", help_, [_line(f"{key}_total", snap.get(key, 0))])
    life = snap.get("draft_policy", {})
    family("draft_tokens_total", "counter", "draft tokens proposed and accepted",
           [_line("draft_tokens_total", life.get(k, 0), {"kind": k}) for k in ("proposed", "accepted")])
    family("requests", "gauge", "requests by state", [_line("requests", snap.get(k, 0), {"state": s})
                                                       for k, s in (("queued", "queued"), ("prefilling", "prefill"), ("active", "decode"))])
    kv = snap.get("kv", {})
    family("kv_pages", "gauge", "KV pages", [_line("kv_pages", kv.get("total_pages", 0), {"kind": "total"}),
                                              _line("kv_pages", kv.get("leased_pages", 0), {"kind": "leased"})])
    family("uptime_seconds", "gauge", "seconds since the server started", [_line("uptime_seconds", round(time.time() - state.started, 1))])
    family("ready", "gauge", "1 once the engine is built", [_line("ready", int(state.sched.ready.is_set()))])
    from ..utils.memory_ledger import LEDGER
    rep = LEDGER.report()
    if rep["by_kind"]:
        family("memory_tracked_bytes", "gauge", "device bytes the ledger accounts for, by kind",
               [_line("memory_tracked_bytes", v, {"kind": k}) for k, v in sorted(rep["by_kind"].items())])
    rows = [_line("memory_untracked_bytes", r["untracked"], {"device": d}) for d, r in rep["devices"].items() if r.get("untracked") is not None]
    if rows:
        family("memory_untracked_bytes", "gauge", "bytes in use on a device that the ledger does not account for", rows)
    try:
        from ..utils.thermal import monitor
        latest = monitor().latest()
    except Exception:                                          # noqa: BLE001 - telemetry never fails a scrape
        latest = {}
    if latest:
        family("gpu_sm_clock_mhz", "gauge", "SM clock", [_line("gpu_sm_clock_mhz", s["sm_mhz"], {"gpu": g}) for g, s in sorted(latest.items())])
        family("gpu_power_watts", "gauge", "board power", [_line("gpu_power_watts", s["power_w"], {"gpu": g}) for g, s in sorted(latest.items())])
        family("gpu_temperature_celsius", "gauge", "GPU temperature", [_line("gpu_temperature_celsius", s["temp_c"], {"gpu": g}) for g, s in sorted(latest.items())])
        family("gpu_throttle_reason", "gauge", "1 while a throttle reason is active",
               [_line("gpu_throttle_reason", 1, {"gpu": g, "reason": r}) for g, s in sorted(latest.items()) for r in s["reason_names"]] or
               [_line("gpu_throttle_reason", 0, {"gpu": g, "reason": "none"}) for g in sorted(latest)])
    return "\n".join(out) + "\n"
