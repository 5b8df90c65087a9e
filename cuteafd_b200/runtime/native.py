"""ctypes front end of libcuteafd_rt.so: the C++ page pool, KV reserve, repeat guard, wire checksum and sampler.

``make_pool`` and ``make_reserve`` are what the backends and the scheduler construct: the C++ page pool and banker's-rule
reserve when the library loads (the default), the Python classes otherwise (or with ``CUTEAFD_NATIVE_RT=0``).  Same
behaviour either way; the tests drive both with identical random workloads.
"""
from __future__ import annotations

import ctypes as C

from .._native import lib as _n

_sigs_done = False


def _lib():
    global _sigs_done
    L = _n.rt_lib()
    if not _sigs_done:
        P, I, IP = C.c_void_p, C.c_int, C.POINTER(C.c_int)
        def sig(name, args, res=I):
            f = getattr(L, name); f.argtypes, f.restype = args, res
        sig("cafd_pool_new", [I], P); sig("cafd_pool_free", [P], None); sig("cafd_pool_free_pages", [P])
        sig("cafd_pool_alloc", [P]); sig("cafd_pool_retain", [P, I]); sig("cafd_pool_release", [P, I]); sig("cafd_pool_refs", [P, I])
        sig("cafd_seq_new", [P]); sig("cafd_seq_reserve", [P, I, I, IP, IP]); sig("cafd_seq_fork", [P, I, I])
        sig("cafd_seq_truncate", [P, I, I]); sig("cafd_seq_free", [P, I]); sig("cafd_seq_set_len", [P, I, I]); sig("cafd_seq_len", [P, I])
        sig("cafd_seq_num_pages", [P, I]); sig("cafd_seq_pages", [P, I, IP, I]); sig("cafd_seq_slots", [P, I, I, I, IP])
        sig("cafd_reserve_total", [P]); sig("cafd_reserve_count", [P]); sig("cafd_reserve_needs_top_up", [P, I, I])
        sig("cafd_reserve_new", [I, I], P); sig("cafd_reserve_free", [P], None); sig("cafd_reserve_lease", [P, I, I, I, I])
        sig("cafd_reserve_top_up", [P, I]); sig("cafd_reserve_release", [P, I]); sig("cafd_reserve_leased", [P])
        sig("cafd_sample_token", [C.POINTER(C.c_float), I, C.POINTER(C.c_uint8), C.c_float, C.c_float, I, C.c_float, C.c_uint64, C.c_uint64, I, C.c_float])
        sig("cafd_sample_uniform", [C.c_uint64, C.c_uint64], C.c_float)
        sig("cafd_guard_new", [I, I, I, I], P); sig("cafd_guard_free", [P], None); sig("cafd_guard_push", [P, C.c_int32])
        sig("cafd_guard_period", [P]); sig("cafd_guard_pushed", [P], C.c_int64)
        U8P, U32, U64 = C.POINTER(C.c_uint8), C.c_uint32, C.c_uint64
        sig("cafd_wire_crc32", [C.c_char_p, U64], U32)
        sig("cafd_wire_pack_request", [C.c_char_p, I, U32, U64, U32, U32, U32, U32, I, I, U32, U64, U32, C.c_char_p], None)
        sig("cafd_wire_parse_request", [C.c_char_p, IP, C.POINTER(U32), C.POINTER(U64), C.POINTER(U32), C.POINTER(U32), C.POINTER(U32),
                                        C.POINTER(U32), IP, IP, C.POINTER(U32), C.POINTER(U64), C.POINTER(U32), C.c_char_p])
        _sigs_done = True
    return L


class NativeRepeatGuard:
    """C++ twin of ``repeat_guard.RepeatGuard`` (same rules, same firing points); ``push`` costs well under a
    microsecond, which matters when 64 streams emit several tokens per step."""

    def __init__(self, cfg):
        self.L = _lib()
        self.cfg = cfg
        self.h = self.L.cafd_guard_new(cfg.run, cfg.copies, cfg.fast_span, cfg.fast_copies)
        self.hit: dict | None = None

    def __del__(self):
        if getattr(self, "h", None):
            self.L.cafd_guard_free(self.h)
            self.h = None

    @property
    def pushed(self) -> int:
        return self.L.cafd_guard_pushed(self.h)

    def push(self, token: int) -> bool:
        if self.hit is not None:
            return True
        r = self.L.cafd_guard_push(self.h, int(token))
        if r:
            self.hit = {"rule": "fast" if r == 1 else "repeat", "period": self.L.cafd_guard_period(self.h), "at": self.pushed}
            return True
        return False


def wire_crc32(data: bytes) -> int:
    return _lib().cafd_wire_crc32(data, len(data))


def wire_pack_request(kind: int, flags: int, seq: int, layer: int, rows: int, hidden: int, routes: int, dtype: int, reply_dtype: int,
                      unit: int, payload_bytes: int, crc: int, plan: bytes) -> bytes:
    buf = C.create_string_buffer(96)
    _lib().cafd_wire_pack_request(buf, kind, flags, seq, layer, rows, hidden, routes, dtype, reply_dtype, unit, payload_bytes, crc, plan)
    return buf.raw


def wire_parse_request(raw: bytes) -> tuple[int, dict]:
    """-> (status, fields) with the protocol's status codes."""
    I, U32, U64 = C.c_int, C.c_uint32, C.c_uint64
    kind, dt, rdt = I(), I(), I()
    flags, layer, rows, hidden, routes, unit, crc = (U32() for _ in range(7))
    seq, nbytes = U64(), U64()
    plan = C.create_string_buffer(16)
    st = _lib().cafd_wire_parse_request(raw, C.byref(kind), C.byref(flags), C.byref(seq), C.byref(layer), C.byref(rows), C.byref(hidden),
                                        C.byref(routes), C.byref(dt), C.byref(rdt), C.byref(unit), C.byref(nbytes), C.byref(crc), plan)
    return st, {"kind": kind.value, "flags": flags.value, "seq": seq.value, "layer": layer.value, "rows": rows.value,
                "hidden": hidden.value, "routes": routes.value, "dtype": dt.value, "reply_dtype": rdt.value, "unit": unit.value,
                "payload_bytes": nbytes.value, "crc": crc.value, "plan": plan.raw}


class NativePool:
    def __init__(self, num_pages: int):
        self.L = _lib()
        self.h = self.L.cafd_pool_new(num_pages)
        if not self.h:
            raise ValueError("pool needs at least 2 pages")

    def __del__(self):
        if getattr(self, "h", None):
            self.L.cafd_pool_free(self.h)
            self.h = None

    @property
    def free_pages(self) -> int:
        return self.L.cafd_pool_free_pages(self.h)

    def refs(self, page: int) -> int:
        return self.L.cafd_pool_refs(self.h, page)

    def new_seq(self) -> int:
        return self.L.cafd_seq_new(self.h)

    def reserve(self, seq: int, new_len: int) -> tuple[int, tuple[int, int] | None]:
        """Returns (pages added or -1, (src, dst) page copy to perform or None)."""
        a, b = C.c_int(-1), C.c_int(-1)
        n = self.L.cafd_seq_reserve(self.h, seq, new_len, C.byref(a), C.byref(b))
        return n, ((a.value, b.value) if a.value >= 0 else None)

    def fork(self, seq: int, length: int = -1) -> int:
        return self.L.cafd_seq_fork(self.h, seq, length)

    def truncate(self, seq: int, length: int) -> None:
        self.L.cafd_seq_truncate(self.h, seq, length)

    def free(self, seq: int) -> None:
        self.L.cafd_seq_free(self.h, seq)

    def set_len(self, seq: int, n: int) -> None:
        self.L.cafd_seq_set_len(self.h, seq, n)

    def pages(self, seq: int) -> list[int]:
        n = self.L.cafd_seq_num_pages(self.h, seq)
        buf = (C.c_int * max(n, 1))()
        self.L.cafd_seq_pages(self.h, seq, buf, n)
        return list(buf[:n])

    def slots(self, seq: int, start: int, n: int) -> list[int]:
        buf = (C.c_int * max(n, 1))()
        if self.L.cafd_seq_slots(self.h, seq, start, n, buf) != 0:
            raise IndexError("slots outside the reserved pages")
        return list(buf[:n])


class NativeReserve:
    def __init__(self, total_pages: int, chunk_tokens: int = 16384):
        self.L = _lib()
        self.h = self.L.cafd_reserve_new(total_pages, chunk_tokens)

    def __del__(self):
        if getattr(self, "h", None):
            self.L.cafd_reserve_free(self.h)
            self.h = None

    def lease(self, rid: int, prompt: int, max_new: int, shared_pages: int = 0):
        """Truthy when admitted, None when refused (the Python reserve returns the lease record or None)."""
        return True if self.L.cafd_reserve_lease(self.h, rid, prompt, max_new, shared_pages) else None

    def needs_top_up(self, rid: int, next_len_tokens: int) -> bool:
        r = self.L.cafd_reserve_needs_top_up(self.h, rid, next_len_tokens)
        if r < 0:
            raise KeyError(rid)
        return bool(r)

    def note_used(self, rid: int, pages: int) -> None:
        pass

    @property
    def total(self) -> int:
        return self.L.cafd_reserve_total(self.h)

    @property
    def unleased(self) -> int:
        return self.total - self.leased

    def __len__(self) -> int:
        return self.L.cafd_reserve_count(self.h)

    def top_up(self, rid: int) -> bool:
        return bool(self.L.cafd_reserve_top_up(self.h, rid))

    def release(self, rid: int) -> None:
        self.L.cafd_reserve_release(self.h, rid)

    @property
    def leased(self) -> int:
        return self.L.cafd_reserve_leased(self.h)


def sample_token(logits, temperature=0.0, top_p=1.0, top_k=None, min_p=0.0, seed=0, position=0, mask=None, uniform=None) -> int:
    """Native sampler on a float32 CPU tensor row.  Negative return values are row status codes."""
    L = _lib()
    x = logits.detach().float().contiguous().cpu()
    lp = C.cast(x.data_ptr(), C.POINTER(C.c_float))
    mp = None
    if mask is not None:
        m = mask.to("cpu").to(dtype=__import__("torch").uint8).contiguous()
        mp = C.cast(m.data_ptr(), C.POINTER(C.c_uint8))
    return L.cafd_sample_token(lp, x.numel(), mp, temperature, top_p, top_k or 0, min_p, seed, position,
                               int(uniform is not None), float(uniform or 0.0))


def sample_uniform(seed: int, position: int) -> float:
    return float(_lib().cafd_sample_uniform(seed, position))


def enabled() -> bool:
    """Whether the serving path builds its host structures on the C++ library (default: yes when it loads)."""
    import os
    if os.environ.get("CUTEAFD_NATIVE_RT", "1") == "0":
        return False
    try:
        _lib()
        return True
    except OSError:
        return False


def make_reserve(total_pages: int, chunk_tokens: int = 16384):
    if enabled():
        return NativeReserve(total_pages, chunk_tokens)
    from .reserve import KvReserve
    return KvReserve(total_pages, chunk_tokens)


def make_pool(num_pages: int):
    from .paged import NativePagePool, PagePool
    return NativePagePool(num_pages) if enabled() else PagePool(num_pages)
