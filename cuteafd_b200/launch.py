"""Launcher: turn a deployment document (``plan --deployment``) into running ranks, one process per GPU.

``cuteafd launch MODEL`` plans the checkpoint on this box's GPUs, writes the deployment document into the run
directory, starts ``cuteafd serve --deployment FILE`` once per rank with the rendezvous environment of that rank
(RANK / LOCAL_RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT), and supervises them: a rank that exits non-zero takes the
deployment down (the others are signalled by their exact process ids), a SIGINT / SIGTERM to the launcher is handed to
rank 0 first so that it can release the expert ranks and leave the process group in order.  ``cuteafd stop`` ends a
deployment by its pid file.  ``--dry-run`` validates the plan and prints the per-rank commands without starting anything.

Counterpart: the reference's ``run.sh`` / ``stop.sh`` pair, which read a KEY=VALUE configuration (``--config``, ``--set``),
plan, and start the coordinator and the expert workers (run.sh:9-37; scripts/launch/run-family.sh).
"""
from __future__ import annotations

import json
import os
import signal
import subprocess
import sys
import time
from dataclasses import dataclass, field


@dataclass
class RankProcess:
    rank: int
    role: str
    argv: list[str]
    env: dict[str, str]
    log: str = ""
    proc: subprocess.Popen | None = None


@dataclass
class Launch:
    """The processes of one deployment."""
    spec: dict
    run_dir: str
    ranks: list[RankProcess] = field(default_factory=list)
    grace_s: float = 20.0

    @property
    def pid_file(self) -> str:
        return os.path.join(self.run_dir, "launch.json")

    def start(self) -> None:
        os.makedirs(self.run_dir, exist_ok=True)
        try:
            for r in self.ranks:
                out = open(r.log, "ab") if r.log else None
                try:
                    r.proc = subprocess.Popen(r.argv, env={**os.environ, **r.env}, stdout=out, stderr=subprocess.STDOUT if out else None)
                finally:
                    if out is not None:
                        out.close()
        except OSError:
            self.stop(signal.SIGTERM)          # a rank that could not be started: the ones already running do not stay behind
            raise
        with open(self.pid_file, "w") as f:
            json.dump({"launcher": os.getpid(), "plan_hash": self.spec.get("plan_hash"),
                       "ranks": [{"rank": r.rank, "role": r.role, "pid": r.proc.pid, "log": r.log} for r in self.ranks]}, f, indent=1)

    def poll(self) -> dict[int, int]:
        """Exit codes of the ranks that have ended."""
        return {r.rank: r.proc.returncode for r in self.ranks if r.proc is not None and r.proc.poll() is not None}

    def stop(self, first_signal: int = signal.SIGINT) -> None:
        """Rank 0 first (it shuts the group down), then whoever is left after the grace period."""
        live = [r for r in self.ranks if r.proc is not None and r.proc.poll() is None]
        head = [r for r in live if r.rank == 0]
        for r in head or live:
            _signal(r.proc.pid, first_signal)
        t0 = time.monotonic()
        while time.monotonic() - t0 < self.grace_s and any(r.proc.poll() is None for r in live):
            time.sleep(0.05)
        for r in live:
            if r.proc.poll() is None:
                _signal(r.proc.pid, signal.SIGTERM)
        t0 = time.monotonic()
        while time.monotonic() - t0 < 5.0 and any(r.proc.poll() is None for r in live):
            time.sleep(0.05)
        for r in live:
            if r.proc.poll() is None:
                _signal(r.proc.pid, signal.SIGKILL)
                r.proc.wait()
        try:
            os.remove(self.pid_file)
        except OSError:
            pass

    def supervise(self, poll_s: float = 0.2) -> int:
        """Block until the deployment ends.  Returns 0 when every rank left cleanly (or after a requested stop), else
        the first failing rank's exit code."""
        stop_requested = []

        def on_signal(signum, _frame):
            stop_requested.append(signum)
        old = {s: signal.signal(s, on_signal) for s in (signal.SIGINT, signal.SIGTERM)}
        try:
            while True:
                ended = self.poll()
                bad = {k: v for k, v in ended.items() if v != 0}
                if bad:
                    rank, rc = sorted(bad.items())[0]
                    print(f"[launch] rank {rank} exited with {rc}: stopping the deployment", file=sys.stderr, flush=True)
                    self.stop()
                    return rc if rc > 0 else 1
                if len(ended) == len(self.ranks):
                    try:
                        os.remove(self.pid_file)
                    except OSError:
                        pass
                    return 0
                if stop_requested:
                    self.stop()
                    return 0
                time.sleep(poll_s)
        finally:
            for s, h in old.items():
                signal.signal(s, h)


def _signal(pid: int, sig: int) -> None:
    try:
        os.kill(pid, sig)
    except ProcessLookupError:
        pass


def rank_env(spec: dict, entry: dict) -> dict[str, str]:
    rv = spec.get("rendezvous", {})
    return {"RANK": str(entry["rank"]), "LOCAL_RANK": str(entry["device"]), "WORLD_SIZE": str(spec["world_size"]),
            "MASTER_ADDR": str(rv.get("master_addr", "127.0.0.1")), "MASTER_PORT": str(rv.get("master_port", 29500))}


def serve_argv(spec_path: str, spec: dict, entry: dict, serve_args: list[str]) -> list[str]:
    """Every rank runs ``serve``: rank 0 builds the attention half and the HTTP server, an expert rank builds its
    expert range and serves announced steps until rank 0 releases it."""
    return [sys.executable, "-m", "cuteafd_b200.cli", "serve", "--snapshot", spec["source"], "--deployment", spec_path, *serve_args]


def build_launch(spec: dict, run_dir: str, serve_args: list[str], argv_for=serve_argv) -> Launch:
    validate(spec)
    os.makedirs(run_dir, exist_ok=True)
    spec_path = os.path.join(run_dir, "deployment.json")
    with open(spec_path, "w") as f:
        json.dump(spec, f, indent=1)
    L = Launch(spec, run_dir)
    for e in spec["ranks"]:
        L.ranks.append(RankProcess(e["rank"], e["role"], argv_for(spec_path, spec, e, serve_args), rank_env(spec, e),
                                   log=os.path.join(run_dir, f"rank{e['rank']}.log")))
    return L


def validate(spec: dict) -> None:
    """Refuse a document this launcher cannot start: ranks numbered 0..world-1, one device each, rank 0 an attention
    rank, expert ranges that tile the expert ids without overlap, and the hash the planner stamped."""
    import hashlib
    ranks = spec.get("ranks") or []
    if [e.get("rank") for e in ranks] != list(range(spec.get("world_size", -1))):
        raise ValueError("deployment: ranks must be numbered 0..world_size-1 in order")
    if len({e["device"] for e in ranks}) != len(ranks):
        raise ValueError("deployment: two ranks share a device")
    if not ranks or "attention" not in ranks[0]["role"]:
        raise ValueError("deployment: rank 0 must be an attention rank")
    spans = sorted(tuple(e["experts"]) for e in ranks if e.get("experts"))
    for (a0, a1), (b0, b1) in zip(spans, spans[1:]):
        if b0 != a1:
            raise ValueError(f"deployment: expert ranges [{a0}:{a1}) and [{b0}:{b1}) do not tile the expert ids")
    if "plan_hash" in spec:
        body = {k: v for k, v in spec.items() if k != "plan_hash"}
        if hashlib.sha256(json.dumps(body, sort_keys=True).encode()).hexdigest()[:16] != spec["plan_hash"]:
            raise ValueError("deployment: plan_hash does not match the document (edited after planning?)")


def describe(L: Launch) -> str:
    lines = [f"deployment {L.spec.get('plan_hash', '?')}: {L.spec.get('layout', '')} ({L.spec['world_size']} ranks)"]
    for r in L.ranks:
        env = " ".join(f"{k}={v}" for k, v in r.env.items())
        lines.append(f"  rank {r.rank} [{r.role}] {env} {' '.join(r.argv)}")
    return "\n".join(lines)


def stop_by_pid_file(path: str, grace_s: float = 20.0) -> int:
    """End a running deployment: the launcher if it is alive (it stops its ranks in order), else the ranks."""
    with open(path) as f:
        doc = json.load(f)
    launcher = doc.get("launcher")
    if launcher and _alive(launcher):
        _signal(launcher, signal.SIGTERM)
        t0 = time.monotonic()
        while time.monotonic() - t0 < grace_s + 10 and _alive(launcher):
            time.sleep(0.1)
        return 0 if not _alive(launcher) else 1
    for r in sorted(doc.get("ranks", []), key=lambda r: r["rank"]):
        _signal(r["pid"], signal.SIGINT if r["rank"] == 0 else signal.SIGTERM)
    return 0


def _alive(pid: int) -> bool:
    try:
        os.kill(pid, 0)
        return True
    except (ProcessLookupError, PermissionError):
        return False
