"""ctypes bindings of libcuteafd_b200.so (CUDA kernels) and libcuteafd_rt.so (host runtime)."""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import build

_lock = threading.Lock()
_cuda = None
_rt = None

c_void_p, c_int, c_float, c_u32p = C.c_void_p, C.c_int, C.c_float, C.c_void_p


class GemmArgs(C.Structure):
    _fields_ = [
        ("w0", C.c_void_p), ("w1", C.c_void_p), ("x", C.c_void_p), ("out", C.c_void_p),
        ("residual", C.c_void_p), ("row_scale", C.c_void_p), ("row_dst", C.c_void_p),
        ("tile_expert", C.c_void_p), ("tile_row0", C.c_void_p), ("num_x_tiles", C.c_void_p),
        ("w_scale", C.c_void_p), ("x_scale", C.c_void_p), ("w_scale1", C.c_void_p),
        ("wait_flag", C.c_void_p), ("epoch", C.c_void_p), ("done_counter", C.c_void_p),
        ("signal_flag", C.c_void_p), ("status", C.c_void_p),
        ("splitk_scratch", C.c_void_p), ("splitk_tickets", C.c_void_p),
        ("splitk_scratch_floats", C.c_longlong), ("splitk_ticket_count", C.c_int),
        ("w_rows_total", C.c_longlong), ("x_rows_total", C.c_longlong),
        ("k", C.c_int), ("n_features", C.c_int), ("x_rows", C.c_int), ("ldo", C.c_int),
        ("w_rows_per_expert", C.c_int), ("w1_row_offset", C.c_int), ("max_x_tiles", C.c_int),
        ("swap", C.c_int), ("dual", C.c_int), ("bx", C.c_int), ("out_f32", C.c_int), ("fp8", C.c_int),
        ("num_sms", C.c_int),
        ("rs_ranks", C.c_int), ("rs_rows_per_rank", C.c_int), ("rs_my_rank", C.c_int), ("n_signal_flags", C.c_int),
        ("n_wait_flags", C.c_int), ("reserved0", C.c_int),
        ("rs_out", C.c_void_p * 8), ("signal_flags", C.c_void_p * 8),
    ]


MAX_RANKS = 8
# one setter per translation unit that waits (each holds its own copy of the limit)
WAIT_LIMIT_SETTERS = ("cafd_gemm_set_wait_limit_ns", "cafd_moe_set_wait_limit_ns", "cafd_attn_set_wait_limit_ns",
                      "cafd_gemm_fp8_set_wait_limit_ns", "cafd_tp_set_wait_limit_ns", "cafd_mla_set_wait_limit_ns",
                      "cafd_indexer_set_wait_limit_ns", "cafd_gemm_w4_set_wait_limit_ns", "cafd_gemm_exl3_set_wait_limit_ns",
                      "cafd_decode_step_set_wait_limit_ns")


BOUNDS_UNITS = ("cafd_moe", "cafd_tp")        # translation units with checked peer-store sites
BOUNDS_SITES = {1: "plan+dispatch: slab row", 2: "plan+dispatch: owner rank", 3: "dispatch: slab row", 4: "dispatch: owner rank",
                6: "head exchange: table row", 7: "head exchange: rank"}


def bounds_check_enabled() -> bool:
    lib = cuda_lib()
    return all(getattr(lib, f"{tu}_bounds_check_enabled")() == 1 for tu in BOUNDS_UNITS)


def take_bad_indices() -> list[tuple[str, int]]:
    """Records the bounds-check build left since the last call: (site, offending index).  Synchronises the device."""
    lib, out = cuda_lib(), []
    for tu in BOUNDS_UNITS:
        v = C.c_ulonglong(0)
        check(getattr(lib, f"{tu}_take_bad_index")(C.byref(v)), f"{tu}_take_bad_index")
        if v.value:
            idx = v.value & 0xffffffffffff
            if idx >= 1 << 47:
                idx -= 1 << 48
            out.append((BOUNDS_SITES.get((v.value >> 48) & 0x7fff, "?"), idx))
    return out


class MoeLayout(C.Structure):
    _fields_ = [
        ("n_ranks", C.c_int), ("expert_lo", C.c_int * (MAX_RANKS + 1)),
        ("slab", C.c_void_p * MAX_RANKS), ("meta", C.c_void_p * MAX_RANKS), ("flag", C.c_void_p * MAX_RANKS),
        ("max_tiles", C.c_int), ("max_rows", C.c_int),
        ("fp8", C.c_int), ("slab_q", C.c_void_p * MAX_RANKS), ("slab_s", C.c_void_p * MAX_RANKS),
    ]


class TpReduceArgs(C.Structure):
    _fields_ = [
        ("partials", C.c_void_p), ("residual", C.c_void_p), ("norm_w", C.c_void_p), ("x_out", C.c_void_p * 8),
        ("rs_flags", C.c_void_p), ("ag_flags", C.c_void_p * 8), ("epoch", C.c_void_p), ("done_counter", C.c_void_p),
        ("status", C.c_void_p), ("ranks", C.c_int), ("my_rank", C.c_int), ("rows_per_rank", C.c_int),
        ("rows_valid", C.c_int), ("N", C.c_int), ("eps", C.c_float), ("n_sum", C.c_int), ("n_wait", C.c_int),
    ]


class TpHeadArgs(C.Structure):
    _fields_ = [
        ("cand_v", C.c_void_p), ("cand_i", C.c_void_p), ("table_out", C.c_void_p * 8), ("table_in", C.c_void_p),
        ("flags_out", C.c_void_p * 8), ("flags_in", C.c_void_p), ("epoch", C.c_void_p), ("done_counter", C.c_void_p),
        ("status", C.c_void_p), ("out", C.c_void_p), ("ranks", C.c_int), ("my_rank", C.c_int), ("max_rows", C.c_int),
        ("T", C.c_int), ("slices", C.c_int), ("lo", C.c_int),
    ]


def _sig(lib, name, argtypes, restype=C.c_int):
    fn = getattr(lib, name)
    fn.argtypes = argtypes
    fn.restype = restype
    return fn


def cuda_lib():
    """Load (building first when the shared object is absent) the CUDA kernel library."""
    global _cuda
    with _lock:
        if _cuda is not None:
            return _cuda
        # CAFD_BOUNDS_CHECK=1: the library whose peer-store paths check every index before the access
        checked = os.environ.get("CAFD_BOUNDS_CHECK", "") == "1"
        path = build.CHECK_LIB if checked else build.CUDA_LIB
        if not os.path.exists(path):
            build.build_check() if checked else build.build_cuda()
        lib = C.CDLL(path)
        P, I, F = C.c_void_p, C.c_int, C.c_float
        _sig(lib, "cafd_gemm", [C.POINTER(GemmArgs), P])
        _sig(lib, "cafd_gemm_fp8", [C.POINTER(GemmArgs), P])
        _sig(lib, "cafd_quant_rows_fp8", [P, P, P, I, I, I, P])
        for n in WAIT_LIMIT_SETTERS:
            _sig(lib, n, [C.c_ulonglong])
        _sig(lib, "cafd_embed", [P, P, P, I, I, I, P])
        _sig(lib, "cafd_rmsnorm", [P, P, P, P, I, I, F, P])
        _sig(lib, "cafd_qk_rope_kv", [P, P, P, P, P, P, P, P, P, I, I, I, I, F, I, P, I, P])
        _sig(lib, "cafd_argmax", [P, P, P, I, I, I, P])
        _sig(lib, "cafd_argmax_slices", [])
        _sig(lib, "cafd_bump_epoch", [P, P])
        _sig(lib, "cafd_decode_advance", [P, P, P, P, P, P, I, I, I, P])
        _sig(lib, "cafd_route_topk", [P, P, P, P, I, I, I, I, I, I, I, F, P])
        _sig(lib, "cafd_moe_meta_ints", [I, I])
        _sig(lib, "cafd_wait_flag", [P, P, P, P])
        _sig(lib, "cafd_tp_reduce_norm_gather", [C.POINTER(TpReduceArgs), P])
        _sig(lib, "cafd_tp_signal", [P, I, P, P])
        _sig(lib, "cafd_tp_head_pick", [C.POINTER(TpHeadArgs), P])
        for tu in BOUNDS_UNITS:
            _sig(lib, f"{tu}_bounds_check_enabled", [])
            _sig(lib, f"{tu}_take_bad_index", [P])
        _sig(lib, "cafd_argmax_candidates", [P, P, P, I, I, I, P])
        _sig(lib, "cafd_moe_plan", [P, I, I, I, I, C.POINTER(MoeLayout), P, P, P, P])
        _sig(lib, "cafd_moe_plan_wide", [P, I, I, I, I, C.POINTER(MoeLayout), P, P, P, P, P])
        _sig(lib, "cafd_moe_plan_wide_ints", [I, I])
        _sig(lib, "cafd_moe_plan_dispatch", [P, I, I, I, I, C.POINTER(MoeLayout), P, P, P, P, I, P, P])
        _sig(lib, "cafd_norm_route", [P, P, F, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, P])
        _sig(lib, "cafd_moe_combine_norm", [P, P, P, P, P, I, I, I, P, I, P, P, P, F, P, P])
        _sig(lib, "cafd_moe_dispatch", [P, P, P, I, I, I, C.POINTER(MoeLayout), P, P, P])
        _sig(lib, "cafd_moe_combine", [P, P, P, P, P, I, I, I, P, I, P, P, P])
        _sig(lib, "cafd_attn_decode_scratch_floats", [I, I, I, I], C.c_longlong)
        _sig(lib, "cafd_attn_decode", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, F, I, P])
        _sig(lib, "cafd_attn_decode_partial", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, I, F, P])
        _sig(lib, "cafd_attn_merge", [P, P, P, I, I, I, I, I, P])
        _sig(lib, "cafd_set_fixed_kv_split", [I])
        _sig(lib, "cafd_fixed_kv_split", [])
        _sig(lib, "cafd_attn_prefill", [P, P, P, P, P, P, P, P, I, I, I, I, I, I, I, I, F, I, P])
        _sig(lib, "cafd_mla_scratch_floats", [I, I], C.c_longlong)
        _sig(lib, "cafd_mla_attention", [P, P, P, P, P, P, P, P, P, P, C.c_longlong, I, I, I, I, I, I, F, P, I, P])
        _sig(lib, "cafd_indexer_scores", [P, P, P, I, F, P, P, P, P, P, P, P, C.c_longlong, I, I, I, I, I, I, P])
        _sig(lib, "cafd_index_topk", [P, I, P, P, P, I, I, I, P, P])
        _sig(lib, "cafd_index_k_store", [P, I, P, P, I, P])
        _sig(lib, "cafd_mla_prep_a", [P, I, I, P, P, P, P, P, P, P, I, F, I, P, P])
        _sig(lib, "cafd_mla_prep_a_fp8", [P, I, I, P, P, P, P, P, P, P, I, F, I, P, P])
        _sig(lib, "cafd_mla_fp8_gather", [P, P, I, P, I, P, P, P, P, I, P, P])
        _sig(lib, "cafd_mla_attention_partial", [P, P, P, P, P, P, P, P, P, I, I, P, C.c_longlong, I, I, I, I, I, F, P])
        _sig(lib, "cafd_mla_merge", [P, P, P, P, P, I, I, I, I, P])
        _sig(lib, "cafd_mla_attention_gathered", [P, P, P, P, P, P, P, P, P, P, C.c_longlong, I, I, I, I, I, F, P, I, P])
        _sig(lib, "cafd_attn_prefill_mla", [P, I, P, I, I, P, P, C.c_longlong, P, P, P, P, P, P, P, I, I, I, I, I, I, F, P])
        _sig(lib, "cafd_gemm_w4", [C.POINTER(GemmArgs), I, P, P, P])
        _sig(lib, "cafd_w4_dequant", [P, P, P, P, C.c_longlong, I, I, I, P])
        _sig(lib, "cafd_fp8_dequant_block128", [P, P, P, C.c_longlong, I, P])
        _sig(lib, "cafd_gemm_exl3", [P, I, P, P, P, P, P, I, P, P, P, I, I, I, I, I, I, P])
        _sig(lib, "cafd_sample_rows", [P, I, I, P, P, I, P, P, P])
        _sig(lib, "cafd_accept_prefix", [P, P, P, I, P, P, P])
        _sig(lib, "cafd_mla_q_split", [P, I, P, P, P, P, I, I, I, I, P])
        _sig(lib, "cafd_mla_small_rows", [])
        _sig(lib, "cafd_mla_absorb_small", [P, I, P, P, P, P, I, I, I, P])
        _sig(lib, "cafd_mla_unabsorb_small", [P, I, P, P, I, I, P])
        _cuda = lib
        return lib


def rt_lib():
    """Load the host runtime library (C++; no CUDA needed)."""
    global _rt
    with _lock:
        if _rt is not None:
            return _rt
        path = build.RT_LIB
        if not os.path.exists(path):
            build.build_rt()
        _rt = C.CDLL(path)
        return _rt


def loaded_libraries() -> list[str]:
    return [p for p, l in ((build.CUDA_LIB, _cuda), (build.RT_LIB, _rt)) if l is not None]


class NativeError(RuntimeError):
    pass


def check(rc: int, what: str) -> None:
    if rc != 0:
        raise NativeError(f"{what} failed with code {rc}")
