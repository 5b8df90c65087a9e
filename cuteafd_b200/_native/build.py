"""In-tree build of the native libraries.

``libcuteafd_b200.so``  CUDA kernels for sm_100a (nvcc, one object per .cu, plain C ABI)
``libcuteafd_b200_chk.so``  the same kernels compiled with -DCAFD_BOUNDS_CHECK: indices that address peer buffers are
                        checked before the access (loaded instead of the first when CAFD_BOUNDS_CHECK=1)
``libcuteafd_rt.so``    host runtime in C++ (page pool, radix prefix index, sampler oracle, ...)

Both are loaded with ctypes; neither links against Python or libtorch, so they compile in seconds
and load on a machine without a GPU.  The reference builds its native layer with CMake for
sm_120/sm_121 (native/CMakeLists.txt:122,475-479); here the only target is sm_100a.
"""
from __future__ import annotations

import hashlib
import os
import shutil
import subprocess
import sys
from concurrent.futures import ThreadPoolExecutor

HERE = os.path.dirname(os.path.abspath(__file__))
CSRC = os.path.join(os.path.dirname(HERE), "csrc")
OBJ = os.path.join(HERE, "build")
CUDA_LIB = os.path.join(HERE, "libcuteafd_b200.so")
CHECK_LIB = os.path.join(HERE, "libcuteafd_b200_chk.so")
CHECK_SOURCES = ("moe.cu", "tp_collective.cu")     # translation units that carry checked sites; the rest are shared objects
RT_LIB = os.path.join(HERE, "libcuteafd_rt.so")

NVCC_FLAGS = ["-gencode", "arch=compute_100a,code=sm_100a", "-lineinfo", "-O3", "-std=c++17",
              "-Xcompiler", "-fPIC", "-Xptxas", "-v", "--expt-relaxed-constexpr"]
CXX_FLAGS = ["-O2", "-std=c++17", "-fPIC", "-Wall", "-pthread", "-fwrapv"]


def _nvcc() -> str:
    for c in (os.environ.get("NVCC"), shutil.which("nvcc"), "/usr/local/cuda/bin/nvcc"):
        if c and os.path.exists(c):
            return c
    raise RuntimeError("nvcc not found")


def _digest(paths: list[str], extra: str) -> str:
    h = hashlib.sha256(extra.encode())
    for p in sorted(paths):
        with open(p, "rb") as f:
            h.update(p.encode() + b"\0" + f.read())
    return h.hexdigest()


def _headers() -> list[str]:
    out = []
    for root, _, files in os.walk(CSRC):
        out += [os.path.join(root, f) for f in files if f.endswith((".h", ".cuh", ".hpp"))]
    return out


def _compile_one(cmd: list[str], log_path: str) -> None:
    r = subprocess.run(cmd, capture_output=True, text=True)
    with open(log_path, "w") as f:
        f.write(" ".join(cmd) + "\n" + r.stdout + r.stderr)
    if r.returncode != 0:
        raise RuntimeError(f"compile failed: {' '.join(cmd)}\n{r.stdout}\n{r.stderr}")


def build_cuda(force: bool = False, verbose: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    srcs = sorted(os.path.join(CSRC, f) for f in os.listdir(CSRC) if f.endswith(".cu"))
    hdr_digest = _digest(_headers(), " ".join(NVCC_FLAGS))
    nvcc = _nvcc()
    jobs, objs = [], []
    for s in srcs:
        o = os.path.join(OBJ, os.path.basename(s)[:-3] + ".o")
        stamp = o + ".sha"
        d = _digest([s], hdr_digest)
        objs.append(o)
        if not force and os.path.exists(o) and os.path.exists(stamp) and open(stamp).read() == d:
            continue
        jobs.append((s, o, stamp, d))
    if jobs:
        with ThreadPoolExecutor(max_workers=min(8, len(jobs))) as ex:
            futs = [ex.submit(_compile_one, [nvcc, *NVCC_FLAGS, "-I", CSRC, "-c", s, "-o", o], o + ".log")
                    for s, o, _, _ in jobs]
            for f in futs:
                f.result()
        for _, o, stamp, d in jobs:
            with open(stamp, "w") as f:
                f.write(d)
        if verbose:
            for _, o, _, _ in jobs:
                sys.stdout.write(open(o + ".log").read())
    if jobs or not os.path.exists(CUDA_LIB):
        _compile_one([nvcc, "-shared", "-o", CUDA_LIB, *objs, "-lcudart"], os.path.join(OBJ, "link.log"))
    return CUDA_LIB


def build_check(force: bool = False) -> str:
    """The bounds-check library: the translation units with checked sites recompiled with -DCAFD_BOUNDS_CHECK, linked
    with the normal objects of everything else."""
    build_cuda(force)
    nvcc = _nvcc()
    flags = [*NVCC_FLAGS, "-DCAFD_BOUNDS_CHECK"]
    hdr_digest = _digest(_headers(), " ".join(flags))
    objs, rebuilt = [], False
    for f in sorted(os.listdir(CSRC)):
        if not f.endswith(".cu"):
            continue
        if f not in CHECK_SOURCES:
            objs.append(os.path.join(OBJ, f[:-3] + ".o"))
            continue
        s, o = os.path.join(CSRC, f), os.path.join(OBJ, f[:-3] + ".chk.o")
        d = _digest([s], hdr_digest)
        objs.append(o)
        if not force and os.path.exists(o) and os.path.exists(o + ".sha") and open(o + ".sha").read() == d:
            continue
        _compile_one([nvcc, *flags, "-I", CSRC, "-c", s, "-o", o], o + ".log")
        with open(o + ".sha", "w") as fh:
            fh.write(d)
        rebuilt = True
    if rebuilt or not os.path.exists(CHECK_LIB) or os.path.getmtime(CHECK_LIB) < os.path.getmtime(CUDA_LIB):
        _compile_one([nvcc, "-shared", "-o", CHECK_LIB, *objs, "-lcudart"], os.path.join(OBJ, "link_chk.log"))
    return CHECK_LIB


def build_rt(force: bool = False) -> str:
    os.makedirs(OBJ, exist_ok=True)
    rt_dir = os.path.join(CSRC, "rt")
    srcs = sorted(os.path.join(rt_dir, f) for f in os.listdir(rt_dir) if f.endswith(".cc")) if os.path.isdir(rt_dir) else []
    if not srcs:
        return ""
    hdrs = [os.path.join(rt_dir, f) for f in os.listdir(rt_dir) if f.endswith(".h")]
    d = _digest(srcs + hdrs, " ".join(CXX_FLAGS))
    stamp = RT_LIB + ".sha"
    if not force and os.path.exists(RT_LIB) and os.path.exists(stamp) and open(stamp).read() == d:
        return RT_LIB
    _compile_one(["g++", *CXX_FLAGS, "-shared", "-o", RT_LIB, *srcs, "-I", rt_dir], os.path.join(OBJ, "rt.log"))
    with open(stamp, "w") as f:
        f.write(d)
    return RT_LIB


def build_all(force: bool = False, verbose: bool = False) -> tuple[str, ...]:
    return build_cuda(force, verbose), build_check(force), build_rt(force)


if __name__ == "__main__":
    libs = build_all(force="--force" in sys.argv, verbose="-v" in sys.argv)
    print("built:", *libs)
