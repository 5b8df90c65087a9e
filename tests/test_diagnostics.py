"""Stack dumps, stall watchdog and host heap monitor (host only)."""
import os
import signal
import threading
import time

from cuteafd_b200.utils.diagnostics import HostHeapMonitor, StallWatchdog, format_stacks, install_stack_dump, resident_bytes


def test_stack_dump_names_threads_and_signal_writes_file(tmp_path):
    ev = threading.Event()
    t = threading.Thread(target=ev.wait, name="parked-worker", daemon=True)
    t.start()
    text = format_stacks()
    assert "parked-worker" in text and "MainThread" in text and "ev.wait" not in text.split("parked-worker")[0]
    path = str(tmp_path / "stacks.txt")
    assert install_stack_dump(path)
    os.kill(os.getpid(), signal.SIGUSR1)
    for _ in range(100):
        if os.path.exists(path) and "parked-worker" in open(path).read():
            break
        time.sleep(0.02)
    assert "parked-worker" in open(path).read()
    ev.set()
    signal.signal(signal.SIGUSR1, signal.SIG_DFL)


def test_watchdog_dumps_once_per_stall_and_only_when_busy(tmp_path):
    now = [0.0]
    wd = StallWatchdog(limit_s=5.0, path=str(tmp_path / "stall.txt"), clock=lambda: now[0])
    now[0] = 10.0
    assert not wd.check()                       # idle: a quiet loop is not a stall
    wd.busy(3)
    assert wd.check() and wd.stalls == 1
    now[0] = 20.0
    assert not wd.check()                       # still the same stall: one dump
    wd.beat()
    now[0] = 22.0
    assert not wd.check()
    now[0] = 26.0
    assert wd.check() and wd.stalls == 2
    assert open(str(tmp_path / "stall.txt")).read().count("==== stack dump") == 2


def test_host_heap_monitor_warns_once():
    assert resident_bytes() > 0
    vals = iter([1 << 30, 3 << 30, 4 << 30])
    msgs = []
    m = HostHeapMonitor(limit_bytes=2 << 30, pinned=lambda: 1 << 20, read=lambda: next(vals), log=msgs.append)
    assert m.sample()["resident_bytes"] == 1 << 30 and not msgs
    m.sample(); m.sample()
    assert len(msgs) == 1 and m.peak == 4 << 30


def test_prewarm_list_from_a_speculation_trace(tmp_path, capsys):
    """Round geometries counted from the trace, most frequent first, in the shape ``serve --prewarm`` reads; a line cut
    short at the end of the file is skipped."""
    import json

    from cuteafd_b200.cli import main
    from cuteafd_b200.utils.trace import prewarm_from_trace
    p = tmp_path / "t.jsonl"
    rounds = ([{"round": i, "requests": [1, 2], "rows": 2, "kept": [0, 0]} for i in range(5)]
              + [{"round": 9, "requests": [1, 2], "rows": 7, "kept": [4, 1]}] * 3
              + [{"round": 10, "requests": [4], "rows": 1, "kept": [0]}] + [{"other": 1}])
    p.write_text("\n".join(json.dumps(r) for r in rounds) + '\n{"round": 11, "requests": [1')
    doc = prewarm_from_trace(str(p), top=2)
    assert doc["geometries"] == [[2, 2, 1], [2, 7, 5]] and doc["seen"] == {"2,2,1": 5, "2,7,5": 3, "1,1,1": 1} and doc["rounds"] == 9
    assert main(["prewarm", str(p), "--out", str(tmp_path / "pw.json")]) == 0
    assert json.load(open(tmp_path / "pw.json"))["geometries"][0] == [2, 2, 1] and "3 geometries from 9 rounds" in capsys.readouterr().out
    assert main(["prewarm", str(tmp_path / "missing.jsonl")]) == 1
