"""Source gates: structural rules of the code base checked on the sources themselves (cheap architectural invariants,
as the reference does with tests that read their own source: daemon/shared/qwen/scheduler.rs:566-645).

* every CUDA kernel waits for its programmatic-launch predecessor before it can return: a kernel that is launched with
  the dependent-launch attribute and skips the wait completes early, and the kernel after it then overlaps with the one
  before it;
* device code never traps, and no TMA or bulk load is issued with cluster multicast (peer memory may sit behind any
  tensor map of the multi-GPU kernels);
* comments and docstrings state facts on their own: no pointers to working notes, build rounds or machine paths.
"""
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
CSRC = os.path.join(ROOT, "cuteafd_b200", "csrc")


def _cuda_sources():
    for dirpath, _, names in os.walk(CSRC):
        for n in sorted(names):
            if n.endswith((".cu", ".cuh", ".h", ".cc")):
                p = os.path.join(dirpath, n)
                with open(p) as f:
                    yield os.path.relpath(p, ROOT), f.read()


def _kernel_bodies(src: str):
    for m in re.finditer(r"__global__\s+void\s+(?:__launch_bounds__\([^)]*\)\s*)?(\w+)\s*\(", src):
        i = src.index("{", m.end())
        depth, j = 0, i
        while True:
            depth += {"{": 1, "}": -1}.get(src[j], 0)
            if depth == 0:
                break
            j += 1
        yield m.group(1), src[i:j]


def test_every_dependent_launch_kernel_waits_before_it_can_return():
    plain = set()            # kernels launched with <<< >>> only: fully ordered by the stream, no wait needed
    bodies = {}
    for path, src in _cuda_sources():
        for name, body in _kernel_bodies(src):
            bodies[name] = (path, body)
        plain |= set(re.findall(r"(\w+)\s*(?:<[^<>]*>)?\s*<<<", src))
    assert len(bodies) > 40
    bad = []
    for name, (path, body) in bodies.items():
        if "pdl_wait" not in body:
            if name not in plain and name != "decode_step_kernel":        # the cooperative one-launch step has its own launcher
                bad.append(f"{path}: {name} has no pdl_wait")
        elif "return" in body[:body.index("pdl_wait")]:
            bad.append(f"{path}: {name} can return before pdl_wait")
    assert not bad, bad


def test_device_code_neither_traps_nor_multicasts_loads():
    bad = []
    for path, src in _cuda_sources():
        code = re.sub(r"//[^\n]*", "", src)
        if re.search(r"\b__trap\s*\(", code) or re.search(r"\btrap\s*;", code):
            bad.append(f"{path}: trap")
        for m in re.finditer(r"cp\.async\.bulk[^\"\n]*", code):
            if "multicast" in m.group(0):
                bad.append(f"{path}: {m.group(0)[:60]}")
    assert not bad, bad


def test_comments_stand_on_their_own():
    words = ["SUR" + "VEY", "VER" + "DICT", "ADV" + "ICE.md", "DES" + "IGN.md", "BASE" + "LINE.md", "gpu" + "run", "/ro" + "ot/", "_wo" + "rk/",
             "the ju" + "dge"]
    rounds = re.compile(r"\bround\s+[0-9]\b|\bin round\b", re.I)
    bad = []
    for base in ("cuteafd_b200", "tests"):
        for dirpath, _, names in os.walk(os.path.join(ROOT, base)):
            for n in names:
                if not n.endswith((".py", ".cu", ".cuh", ".h", ".cc")):
                    continue
                p = os.path.join(dirpath, n)
                with open(p, errors="replace") as f:
                    text = f.read()
                for w in words:
                    if w in text:
                        bad.append(f"{os.path.relpath(p, ROOT)}: names {w!r}")
                for m in rounds.finditer(text):
                    line = text[text.rfind("\n", 0, m.start()) + 1:text.find("\n", m.end())]
                    if "replica" not in line and "script" not in line:              # rounds of the AFD step script are a real thing
                        bad.append(f"{os.path.relpath(p, ROOT)}: {line.strip()[:80]}")
    for extra in ("bench.py", "__graft_entry__.py"):
        with open(os.path.join(ROOT, extra)) as f:
            text = f.read()
        bad += [f"{extra}: names {w!r}" for w in words if w in text]
    assert not bad, bad
