"""Benchmark reports, cards and the published results table.

A *report* is one accepted (or rejected) benchmark run on one checkpoint and one hardware layout: the panels that ran
with their checks, the headline card numbers (prefill tok/s, time to first token, decode tok/s at each concurrency), the
clock record and the build.  Reports live under ``benchmarks/<family>/<date>-<profile>-<hardware>/report.json`` next to a
rendered ``card.svg`` / ``card.md``.  ``publish`` rebuilds two generated blocks from what is on disk: the results table
in the root README (one row per checkpoint, one column per reference layout, each cell resolved through
``benchmarks/current-matrix.json`` to exactly one accepted report, never "whatever is newest") and the index of every
report in ``benchmarks/README.md``.

Counterpart: rust/crates/cuteafd-bench/src/publish.rs:1-60 (markers, matrix, scan), report.rs (report + check status),
render/ (cards).
"""
from __future__ import annotations

import datetime as _dt
import html
import json
import os
import re
from dataclasses import asdict, dataclass, field

REPORT_SCHEMA = "cuteafd_b200.bench.report/1"
MATRIX_SCHEMA = "cuteafd_b200.bench.matrix/1"
MATRIX_FILE = os.path.join("benchmarks", "current-matrix.json")
RESULTS_BEGIN, RESULTS_END = "<!-- results:begin -->", "<!-- results:end -->"
INDEX_BEGIN, INDEX_END = "<!-- reports:begin -->", "<!-- reports:end -->"
COLUMNS = (("1gpu", "1x B200"), ("8gpu", "8x B200"))       # the reference layouts of the published table
STATUSES = ("current", "held", "pending", "na")
GATING = ("smoke", "cache_exact", "lossless")               # a report with one of these failing is not accepted


@dataclass
class Check:
    name: str
    ok: bool
    detail: str = ""
    gating: bool = True


@dataclass
class Report:
    family: str
    checkpoint: str
    hardware: str                     # e.g. "8gpu-2att-6exp"
    profile: str = "smoke"
    created: str = ""
    build: str = ""
    config: dict = field(default_factory=dict)
    card: dict = field(default_factory=dict)      # prefill_tok_s, ttft_s, decode_tok_s {"1": .., "8": .., "32": ..}
    clocks: dict = field(default_factory=dict)
    checks: list = field(default_factory=list)
    panels: list = field(default_factory=list)
    schema: str = REPORT_SCHEMA

    @property
    def accepted(self) -> bool:
        return all(c["ok"] for c in self.checks if c.get("gating", True)) and not _throttled(self.clocks)

    def dir_name(self) -> str:
        return f"{self.created[:10]}-{_slug(self.profile)}-{_slug(self.checkpoint.split('/')[-1])}-{_slug(self.hardware)}"

    def to_json(self) -> dict:
        return asdict(self)

    @staticmethod
    def from_json(d: dict) -> "Report":
        if d.get("schema") != REPORT_SCHEMA:
            raise ValueError(f"not a {REPORT_SCHEMA} document")
        known = {f for f in Report.__dataclass_fields__}
        extra = set(d) - known
        if extra:
            raise ValueError(f"report: unknown fields {sorted(extra)}")
        return Report(**d)


def _slug(s: str) -> str:
    return re.sub(r"[^a-z0-9]+", "-", s.lower()).strip("-")


def _throttled(clocks: dict) -> bool:
    bad = {"hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown"}
    return bool(bad & set(clocks.get("reasons") or []))


def now() -> str:
    return _dt.datetime.now(_dt.timezone.utc).strftime("%Y-%m-%dT%H:%M:%SZ")


# ---- building reports ------------------------------------------------------------------------------------------
def from_panels(out: dict, *, family: str, checkpoint: str, hardware: str, profile: str = "smoke", build: str = "",
                config: dict | None = None) -> Report:
    """Report of a ``panels.run`` result (panels against a live server)."""
    checks, card = [], {}
    for p in out.get("panels", []):
        checks.append(asdict(Check(p["panel"], bool(p.get("ok")), p.get("error", ""), p["panel"] in GATING)))
        if p["panel"] == "speed" and p.get("ok"):
            card["prefill_tok_s"], card["ttft_s"] = p.get("prefill_tok_s"), p.get("prefill_ttft_s")
            card.setdefault("decode_tok_s", {}).setdefault("1", p.get("c1_decode_tok_s"))
        if p["panel"] == "sweep" and p.get("ok") and "levels" in p:
            card["decode_tok_s"] = {str(k): (v.get("tok_s") if isinstance(v, dict) else v) for k, v in p["levels"].items()}
    th = [p.get("thermal") for p in out.get("panels", []) if p.get("thermal")]
    clocks = {"per_panel": th} if th else {}
    return Report(family, checkpoint, hardware, profile, now(), build, config or {}, card, clocks, checks, out.get("panels", []))


def from_bench_line(line: dict, *, family: str, checkpoint: str, profile: str = "card", build: str = "",
                    hardware: str = "") -> Report:
    """Report of the one-line JSON ``bench.py`` prints (the device-timed card of a random-init checkpoint): its
    ``extra`` carries ``decode_tok_s_c<N>`` per concurrency, ``prefill_tok_s_8k`` and ``ttft_s_8k``."""
    cfg = line.get("config", {})
    extra = line.get("extra", {})
    n = int(line.get("n_gpus", 1))

    def first(*names):
        return next((extra[k] for k in names if extra.get(k) is not None), None)
    decode = {}
    for k, v in extra.items():
        for pre, suf in (("decode_tok_s_c", ""), ("decode_c", "_tok_s")):
            if k.startswith(pre) and k.endswith(suf) and k[len(pre):len(k) - len(suf)].isdigit():
                decode[k[len(pre):len(k) - len(suf)]] = v
    card = {"prefill_tok_s": first("prefill_tok_s_8k", "prefill_tok_s"), "ttft_s": first("ttft_s_8k", "ttft_s"),
            "decode_tok_s": dict(sorted(decode.items(), key=lambda kv: int(kv[0])))}
    if not card["decode_tok_s"]:
        card["decode_tok_s"] = {"headline": line.get("value")}
    checks = [asdict(Check("launches", bool(line.get("gpu_launches")), f"{line.get('gpu_launches')} kernel launches per step")),
              asdict(Check("e2e", bool((line.get("e2e") or {}).get("value")), "end-to-end number with host copies", gating=False))]
    return Report(family, checkpoint, hardware or f"{n}gpu-{_slug(str(cfg.get('parallelism', 'single')))[:40]}", profile, now(), build, cfg, card,
                  line.get("clocks") or {}, checks, [])


def write_report(rep: Report, root: str) -> str:
    """Place a report: ``<root>/benchmarks/<family>/<dir>/{report.json, card.svg, card.md}``.  Returns the directory
    relative to ``root``.  An existing directory is never overwritten."""
    rel = os.path.join("benchmarks", _slug(rep.family).replace("-", "_"), rep.dir_name())
    path = os.path.join(root, rel)
    if os.path.exists(os.path.join(path, "report.json")):
        raise FileExistsError(f"{rel} already holds a report")
    os.makedirs(path, exist_ok=True)
    with open(os.path.join(path, "report.json"), "w") as f:
        json.dump(rep.to_json(), f, indent=1)
    with open(os.path.join(path, "card.svg"), "w") as f:
        f.write(render_card_svg(rep))
    with open(os.path.join(path, "card.md"), "w") as f:
        f.write(render_card_md(rep))
    return rel


# ---- cards --------------------------------------------------------------------------------------------------------
def _fmt(v, unit="") -> str:
    if v is None:
        return "-"
    if isinstance(v, float):
        v = round(v, 3 if v < 10 else 1)
    return f"{v:,}{unit}" if isinstance(v, (int, float)) else f"{v}{unit}"


def card_rows(rep: Report) -> list[tuple[str, str]]:
    rows = [("8K prefill", _fmt(rep.card.get("prefill_tok_s"), " tok/s")), ("time to first token", _fmt(rep.card.get("ttft_s"), " s"))]
    for level, v in sorted((rep.card.get("decode_tok_s") or {}).items(), key=lambda kv: (len(kv[0]), kv[0])):
        rows.append((f"decode C{level}" if level.isdigit() else f"decode {level}", _fmt(v, " tok/s")))
    return rows


def render_card_md(rep: Report) -> str:
    L = [f"# {rep.checkpoint} on {rep.hardware}", "", f"{rep.profile} run of {rep.created}; build `{rep.build or 'unknown'}`; "
         f"{'accepted' if rep.accepted else 'NOT accepted'}.", "", "| metric | value |", "|---|---:|"]
    L += [f"| {k} | {v} |" for k, v in card_rows(rep)]
    L += ["", "| check | status | detail |", "|---|---|---|"]
    L += [f"| {c['name']}{'' if c.get('gating', True) else ' (informational)'} | {'pass' if c['ok'] else 'FAIL'} | {c.get('detail', '')} |"
          for c in rep.checks]
    if rep.clocks:
        L += ["", f"clocks: `{json.dumps(rep.clocks)[:300]}`"]
    return "\n".join(L) + "\n"


def render_card_svg(rep: Report) -> str:
    rows = card_rows(rep)
    h = 96 + 26 * len(rows) + 22 * max(1, len(rep.checks))
    esc = html.escape
    out = [f'<svg xmlns="http://www.w3.org/2000/svg" width="560" height="{h}" font-family="monospace" font-size="14">',
           f'<rect width="560" height="{h}" fill="#10141a"/>',
           f'<text x="16" y="28" fill="#e8edf2" font-size="17">{esc(rep.checkpoint)}</text>',
           f'<text x="16" y="50" fill="#8aa0b4">{esc(rep.hardware)} - {esc(rep.profile)} - {esc(rep.created[:10])} - '
           f'{"accepted" if rep.accepted else "not accepted"}</text>']
    y = 82
    for k, v in rows:
        out.append(f'<text x="16" y="{y}" fill="#8aa0b4">{esc(k)}</text><text x="544" y="{y}" fill="#e8edf2" text-anchor="end">{esc(v)}</text>')
        y += 26
    for c in rep.checks:
        col = "#6cc070" if c["ok"] else "#e0605a"
        out.append(f'<text x="16" y="{y}" fill="{col}">{"pass" if c["ok"] else "FAIL"} {esc(c["name"])}</text>')
        y += 22
    out.append("</svg>")
    return "\n".join(out) + "\n"


# ---- publish -------------------------------------------------------------------------------------------------------
@dataclass
class Placed:
    dir: str
    report: Report


def scan(root: str) -> list[Placed]:
    """Every ``benchmarks/*/*/report.json`` under ``root``, newest first."""
    placed = []
    base = os.path.join(root, "benchmarks")
    if not os.path.isdir(base):
        return placed
    for fam in sorted(os.listdir(base)):
        fdir = os.path.join(base, fam)
        if not os.path.isdir(fdir):
            continue
        for d in sorted(os.listdir(fdir)):
            p = os.path.join(fdir, d, "report.json")
            if os.path.isfile(p):
                with open(p) as f:
                    placed.append(Placed(os.path.join("benchmarks", fam, d), Report.from_json(json.load(f))))
    placed.sort(key=lambda x: (x.report.created, x.dir), reverse=True)
    return placed


def load_matrix(root: str, path: str | None = None) -> dict:
    with open(os.path.join(root, path or MATRIX_FILE)) as f:
        m = json.load(f)
    if m.get("schema") != MATRIX_SCHEMA:
        raise ValueError(f"matrix: schema must be {MATRIX_SCHEMA}")
    seen = set()
    for row in m.get("cells", []):
        extra = set(row) - {"family", "checkpoint"} - {c for c, _ in COLUMNS}
        if extra:
            raise ValueError(f"matrix: unknown keys {sorted(extra)} in row {row.get('checkpoint')}")
        key = (row["family"], row["checkpoint"])
        if key in seen:
            raise ValueError(f"matrix: {key} listed twice")
        seen.add(key)
        for col, _ in COLUMNS:
            cell = row.get(col, "pending")
            cell = {"status": cell} if isinstance(cell, str) else cell
            if cell.get("status") not in STATUSES:
                raise ValueError(f"matrix: {key} {col}: status must be one of {STATUSES}")
            if cell["status"] == "current" and not cell.get("report"):
                raise ValueError(f"matrix: {key} {col}: a current cell names its report directory")
            if cell["status"] != "current" and not cell.get("reason"):
                raise ValueError(f"matrix: {key} {col}: a {cell['status']} cell gives its reason")
            row[col] = cell
    return m


def resolve(matrix: dict, placed: list[Placed]) -> list[dict]:
    """Matrix rows with every current cell resolved to its accepted report (a missing or rejected one is an error)."""
    by_dir = {p.dir: p.report for p in placed}
    rows = []
    for row in matrix["cells"]:
        cells = {}
        for col, _ in COLUMNS:
            cell = row[col]
            if cell["status"] == "current":
                rep = by_dir.get(os.path.normpath(cell["report"]))
                if rep is None:
                    raise ValueError(f"matrix: {cell['report']} holds no report")
                if not rep.accepted:
                    raise ValueError(f"matrix: {cell['report']} is not an accepted report")
                if rep.checkpoint != row["checkpoint"]:
                    raise ValueError(f"matrix: {cell['report']} is a report of {rep.checkpoint}, not {row['checkpoint']}")
                cells[col] = {"status": "current", "dir": os.path.normpath(cell["report"]), "report": rep}
            else:
                cells[col] = {"status": cell["status"], "reason": cell["reason"]}
        rows.append({"family": row["family"], "checkpoint": row["checkpoint"], "cells": cells})
    return rows


def _cell_text(cell: dict) -> str:
    if cell["status"] != "current":
        return cell["reason"] if cell["status"] == "na" else f"{cell['status']}: {cell['reason']}"
    rep = cell["report"]
    dec = rep.card.get("decode_tok_s") or {}
    parts = [f"C{k} {_fmt(v)}" for k, v in sorted(dec.items(), key=lambda kv: (len(kv[0]), kv[0])) if k.isdigit()]
    head = " / ".join(parts) or _fmt(next(iter(dec.values()), None))
    tail = f"; prefill {_fmt(rep.card.get('prefill_tok_s'))} tok/s; TTFT {_fmt(rep.card.get('ttft_s'))} s"
    return f"[{head} tok/s{tail}]({cell['dir']}/card.md)"


def results_table(rows: list[dict]) -> str:
    L = ["| checkpoint | " + " | ".join(t for _, t in COLUMNS) + " |", "|---|" + "---|" * len(COLUMNS)]
    for r in rows:
        L.append(f"| {r['checkpoint']} | " + " | ".join(_cell_text(r["cells"][c]) for c, _ in COLUMNS) + " |")
    return "\n".join(L)


def index_table(placed: list[Placed]) -> str:
    L = ["| date | checkpoint | hardware | profile | accepted | report |", "|---|---|---|---|---|---|"]
    for p in placed:
        r = p.report
        L.append(f"| {r.created[:10]} | {r.checkpoint} | {r.hardware} | {r.profile} | {'yes' if r.accepted else 'no'} | "
                 f"[{os.path.basename(p.dir)}]({os.path.relpath(p.dir, 'benchmarks')}/card.md) |")
    return "\n".join(L)


def splice(text: str, begin: str, end: str, body: str) -> str:
    """Replace what stands between the two marker lines; both markers must be there, once, in order."""
    if text.count(begin) != 1 or text.count(end) != 1 or text.index(begin) > text.index(end):
        raise ValueError(f"markers {begin} ... {end} must appear once each, in order")
    a, b = text.index(begin) + len(begin), text.index(end)
    return text[:a] + "\n" + body + "\n" + text[b:]


def publish(root: str, matrix_path: str | None = None, check: bool = False) -> dict:
    """Rebuild the README results table and the benchmarks index.  ``check``: write nothing, report whether the
    committed files are current (for CI)."""
    placed = scan(root)
    rows = resolve(load_matrix(root, matrix_path), placed)
    targets = [(os.path.join(root, "README.md"), RESULTS_BEGIN, RESULTS_END, results_table(rows)),
               (os.path.join(root, "benchmarks", "README.md"), INDEX_BEGIN, INDEX_END, index_table(placed))]
    stale = []
    for path, b, e, body in targets:
        with open(path) as f:
            old = f.read()
        new = splice(old, b, e, body)
        if new != old:
            stale.append(os.path.relpath(path, root))
            if not check:
                with open(path, "w") as f:
                    f.write(new)
    return {"reports": len(placed), "rows": len(rows), "changed": stale, "current": not stale}
