"""Torch-tensor front end of the sm_100a kernels.

Every function launches on the current CUDA stream, allocates nothing beyond its outputs (and
not even those when ``out=`` is given), and raises if the native library is missing: there is no
PyTorch fallback on a GPU box.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from .._native import lib as _n

_status: dict[int, torch.Tensor] = {}
_NUM_SMS: dict[int, int] = {}


def _ptr(t: torch.Tensor | None) -> int | None:
    return None if t is None else t.data_ptr()


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def status_word(device: torch.device | None = None) -> torch.Tensor:
    """Per-device status word: kernels CAS a code into it when a bounded wait runs out."""
    idx = torch.cuda.current_device() if device is None or device.index is None else device.index
    if idx not in _status:
        _status[idx] = torch.zeros(1, dtype=torch.int32, device=f"cuda:{idx}")
    return _status[idx]


def read_status(reset: bool = True) -> int:
    s = status_word()
    v = int(s.item())
    if reset and v:
        s.zero_()
    return v


def num_sms() -> int:
    d = torch.cuda.current_device()
    if d not in _NUM_SMS:
        _NUM_SMS[d] = torch.cuda.get_device_properties(d).multi_processor_count
    return _NUM_SMS[d]


def set_wait_limit_ns(ns: int) -> None:
    """Wall-clock limit of every bounded device wait (default 2 s), for all kernels of the library."""
    L = _n.cuda_lib()
    for name in _n.WAIT_LIMIT_SETTERS:
        _n.check(getattr(L, name)(ns), "set_wait_limit")


# ---- GEMM ------------------------------------------------------------------------------------------
_splitk: dict[tuple[int, int], tuple[torch.Tensor, torch.Tensor]] = {}
_splitk_lane = 0                     # callers running lanes on separate streams switch this
SPLITK_SCRATCH_FLOATS = 8 << 20      # 32 MiB of fp32 partial tiles per (device, stream)
SPLITK_TICKETS = 4096


def splitk_buffers(device: torch.device) -> tuple[torch.Tensor, torch.Tensor]:
    """Scratch + arrival counters for split-K, one set per (device, lane): launches that overlap
    on the GPU (different streams) must not share them; see ``set_splitk_lane``."""
    key = (device.index if device.index is not None else torch.cuda.current_device(), _splitk_lane)
    if key not in _splitk:
        _splitk[key] = (torch.empty(SPLITK_SCRATCH_FLOATS, dtype=torch.float32, device=device),
                        torch.zeros(SPLITK_TICKETS, dtype=torch.int32, device=device))
    return _splitk[key]


def set_splitk_lane(lane: int) -> None:
    global _splitk_lane
    _splitk_lane = lane


def _attach_splitk(a: "_n.GemmArgs", device: torch.device) -> None:
    sc, tk = splitk_buffers(device)
    a.splitk_scratch, a.splitk_tickets = sc.data_ptr(), tk.data_ptr()
    a.splitk_scratch_floats, a.splitk_ticket_count = sc.numel(), tk.numel()

def pick_token_tile(rows: int) -> int:
    """Token tile for the weights-on-M orientation."""
    for b in (16, 32, 64, 128):
        if rows <= b:
            return b
    return 128


def linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor | None = None, *, w_up: torch.Tensor | None = None,
           residual: torch.Tensor | None = None, out_f32: bool = False, swap: bool | None = None,
           split_k: bool = True) -> torch.Tensor:
    """y = x @ w.T (bf16 in, fp32 accumulate).  With ``w_up``: y = silu(x @ w.T) * (x @ w_up.T).

    x [T, K], w [N, K].  ``swap`` picks the orientation (default: weights on M when T <= 128).
    """
    T, K = x.shape
    N = w.shape[0]
    assert x.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x.is_contiguous() and w.is_contiguous()
    assert w.shape[1] == K
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    if T == 0:
        return out
    if swap is None:
        swap = T <= 128
    a = _n.GemmArgs()
    a.w0, a.w1, a.x, a.out = w.data_ptr(), _ptr(w_up), x.data_ptr(), out.data_ptr()
    a.residual = _ptr(residual)
    a.status = status_word(x.device).data_ptr()
    a.w_rows_total, a.x_rows_total = N, T
    a.k, a.n_features, a.x_rows, a.ldo = K, N, T, out.stride(0)
    a.w_rows_per_expert, a.w1_row_offset, a.max_x_tiles = 0, 0, 0
    a.swap, a.dual, a.bx = int(swap), int(w_up is not None), pick_token_tile(T) if swap else 128
    if swap and T > 128:
        a.bx = 128
    a.out_f32, a.fp8, a.num_sms = int(out.dtype == torch.float32), 0, num_sms()
    if swap and split_k:
        _attach_splitk(a, x.device)
    _n.check(_n.cuda_lib().cafd_gemm(C.byref(a), _stream()), "cafd_gemm")
    return out


def grouped_linear(x: torch.Tensor, w: torch.Tensor, out: torch.Tensor, tile_expert: torch.Tensor,
                   tile_row0: torch.Tensor, num_tiles: torch.Tensor, max_tiles: int, tile_rows: int, *,
                   w_up: torch.Tensor | None = None, row_dst: torch.Tensor | None = None,
                   wait_flag: int | None = None, epoch: torch.Tensor | None = None,
                   signal_flag: int | None = None, done_counter: torch.Tensor | None = None,
                   out_ptr: int | None = None, ldo: int | None = None, split_k: bool = True) -> None:
    """Expert-grouped GEMM over an expert-sorted slab.

    x [rows, K] slab, w [E, N, K] stacked expert weights, tiles described by device arrays.
    ``tile_rows`` 128 puts tokens on M (prefill); 16..64 puts weights on M (decode).
    ``out_ptr`` overrides the destination address (a peer GPU's buffer).
    """
    E, N, K = w.shape
    a = _n.GemmArgs()
    a.w0, a.w1, a.x = w.data_ptr(), _ptr(w_up), x.data_ptr()
    a.out = out_ptr if out_ptr is not None else out.data_ptr()
    a.row_dst = _ptr(row_dst)
    a.tile_expert, a.tile_row0, a.num_x_tiles = tile_expert.data_ptr(), tile_row0.data_ptr(), num_tiles.data_ptr()
    a.wait_flag, a.epoch = wait_flag, _ptr(epoch)
    a.signal_flag, a.done_counter = signal_flag, _ptr(done_counter)
    a.status = status_word(x.device).data_ptr()
    a.w_rows_total, a.x_rows_total = E * N, x.shape[0]
    a.k, a.n_features, a.x_rows = K, N, x.shape[0]
    a.ldo = ldo if ldo is not None else out.stride(0)
    a.w_rows_per_expert, a.w1_row_offset, a.max_x_tiles = N, 0, max_tiles
    swap = tile_rows < 128
    a.swap, a.dual, a.bx = int(swap), int(w_up is not None), tile_rows
    a.out_f32, a.fp8, a.num_sms = 0, 0, num_sms()
    if swap and split_k:
        _attach_splitk(a, x.device)
    _n.check(_n.cuda_lib().cafd_gemm(C.byref(a), _stream()), "cafd_gemm(grouped)")


# ---- elementwise -----------------------------------------------------------------------------------
def embed(tokens: torch.Tensor, table: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    T, (V, H) = tokens.shape[0], table.shape
    if out is None:
        out = torch.empty(T, H, dtype=table.dtype, device=table.device)
    _n.check(_n.cuda_lib().cafd_embed(tokens.data_ptr(), table.data_ptr(), out.data_ptr(), T, H, V, _stream()), "embed")
    return out


def rmsnorm(x: torch.Tensor, w: torch.Tensor, eps: float, out: torch.Tensor | None = None) -> torch.Tensor:
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    _n.check(_n.cuda_lib().cafd_rmsnorm(None, x.data_ptr(), w.data_ptr(), out.data_ptr(), T, H, eps, _stream()), "rmsnorm")
    return out


def add_rmsnorm(x: torch.Tensor, residual: torch.Tensor, w: torch.Tensor, eps: float,
                out: torch.Tensor | None = None) -> torch.Tensor:
    """residual += x (in place); returns rmsnorm(residual) * w."""
    T, H = x.shape
    if out is None:
        out = torch.empty_like(x)
    _n.check(_n.cuda_lib().cafd_rmsnorm(x.data_ptr(), residual.data_ptr(), w.data_ptr(), out.data_ptr(), T, H, eps,
                                        _stream()), "add_rmsnorm")
    return out


def qk_rope_kv(qkv: torch.Tensor, q_norm: torch.Tensor | None, k_norm: torch.Tensor | None, inv_freq: torch.Tensor,
               positions: torch.Tensor, slots: torch.Tensor, q_out: torch.Tensor, k_cache: torch.Tensor,
               v_cache: torch.Tensor, Hq: int, Hkv: int, D: int, eps: float, interleaved: bool,
               bias: torch.Tensor | None = None) -> None:
    """q / k head norm (optional), RoPE and the paged K / V write for one step.  ``bias`` [(Hq + 2 Hkv) * D] bf16 is added
    to the fused projection's rows first; the number of rotated dims is twice the length of ``inv_freq`` (128 or 64)."""
    T = qkv.shape[0]
    _n.check(_n.cuda_lib().cafd_qk_rope_kv(qkv.data_ptr(), _ptr(q_norm), _ptr(k_norm), inv_freq.data_ptr(),
                                           positions.data_ptr(), slots.data_ptr(), q_out.data_ptr(), k_cache.data_ptr(),
                                           v_cache.data_ptr(), T, Hq, Hkv, D, eps, int(interleaved), _ptr(bias),
                                           2 * inv_freq.shape[0], _stream()),
             "qk_rope_kv")


_argmax_scratch: dict[int, torch.Tensor] = {}


def argmax(logits: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """Greedy selection per row: ties to the lowest id, NaN never selected."""
    T, V = logits.shape
    if out is None:
        out = torch.empty(T, dtype=torch.int32, device=logits.device)
    L = _n.cuda_lib()
    need = 2 * T * L.cafd_argmax_slices()
    d = logits.device.index or 0
    if d not in _argmax_scratch or _argmax_scratch[d].numel() < need:
        _argmax_scratch[d] = torch.empty(max(need, 2 * 64 * 64), dtype=torch.int32, device=logits.device)
    _n.check(L.cafd_argmax(logits.data_ptr(), out.data_ptr(), _argmax_scratch[d].data_ptr(), T, V, logits.stride(0),
                           _stream()), "argmax")
    return out


def decode_advance(tokens: torch.Tensor, next_tokens: torch.Tensor, positions: torch.Tensor, seq_lens: torch.Tensor,
                   slots: torch.Tensor, page_table: torch.Tensor, page_size: int = 64) -> None:
    """Device-side step bookkeeping: token feedback, position/length +1, next KV slot."""
    S, max_pages = page_table.shape
    _n.check(_n.cuda_lib().cafd_decode_advance(tokens.data_ptr(), next_tokens.data_ptr(), positions.data_ptr(),
                                               seq_lens.data_ptr(), slots.data_ptr(), page_table.data_ptr(), max_pages,
                                               S, page_size, _stream()), "decode_advance")


def bump_epoch(epoch: torch.Tensor) -> None:
    _n.check(_n.cuda_lib().cafd_bump_epoch(epoch.data_ptr(), _stream()), "bump_epoch")


# ---- MoE -------------------------------------------------------------------------------------------
def route_topk(logits: torch.Tensor, top_k: int, scoring: str = "softmax", bias: torch.Tensor | None = None,
               num_groups: int = 1, topk_groups: int = 1, normalize: bool = True, routed_scale: float = 1.0,
               out_idx: torch.Tensor | None = None, out_w: torch.Tensor | None = None):
    T, E = logits.shape
    assert logits.dtype == torch.float32 and logits.is_contiguous()
    if out_idx is None:
        out_idx = torch.empty(T, top_k, dtype=torch.int32, device=logits.device)
    if out_w is None:
        out_w = torch.empty(T, top_k, dtype=torch.float32, device=logits.device)
    _n.check(_n.cuda_lib().cafd_route_topk(logits.data_ptr(), _ptr(bias), out_idx.data_ptr(), out_w.data_ptr(), T, E,
                                           top_k, int(scoring == "sigmoid"), num_groups, topk_groups, int(normalize),
                                           routed_scale, _stream()), "route_topk")
    return out_idx, out_w


def wait_flag(flag_ptr: int, epoch: torch.Tensor) -> None:
    """Stream-ordered bounded wait until *flag >= *epoch (a peer GPU writes the flag)."""
    _n.check(_n.cuda_lib().cafd_wait_flag(flag_ptr, epoch.data_ptr(), status_word(epoch.device).data_ptr(), _stream()), "wait_flag")


def moe_meta_ints(max_tiles: int, max_rows: int) -> int:
    return _n.cuda_lib().cafd_moe_meta_ints(max_tiles, max_rows)


def moe_plan(idx: torch.Tensor, E: int, tile_rows: int, layout: "_n.MoeLayout", dest_row: torch.Tensor,
             expert_count: torch.Tensor | None = None, x: torch.Tensor | None = None, epoch: torch.Tensor | None = None) -> None:
    """Plan the exchange; with ``x`` (and ``epoch``) the same single-block launch also copies the rows into the owners'
    slabs and raises their flags (steps with few rows: saves the dispatch launch)."""
    T, k = idx.shape
    if x is not None:
        _n.check(_n.cuda_lib().cafd_moe_plan_dispatch(idx.data_ptr(), T, k, E, tile_rows, C.byref(layout), dest_row.data_ptr(),
                                                      _ptr(expert_count), status_word(idx.device).data_ptr(), x.data_ptr(),
                                                      x.shape[1], epoch.data_ptr(), _stream()), "moe_plan_dispatch")
        return
    if T * k >= WIDE_PLAN_ENTRIES:
        # prefill-sized step: count / scan / scatter over the whole GPU instead of one block walking every entry
        need = _n.cuda_lib().cafd_moe_plan_wide_ints(T * k, E)
        sc = _plan_scratch.get(idx.device.index)
        if sc is None or sc.numel() < need:
            sc = torch.empty(max(need, 1 << 16), dtype=torch.int32, device=idx.device)
            _plan_scratch[idx.device.index] = sc
        _n.check(_n.cuda_lib().cafd_moe_plan_wide(idx.data_ptr(), T, k, E, tile_rows, C.byref(layout), dest_row.data_ptr(),
                                                  _ptr(expert_count), status_word(idx.device).data_ptr(), sc.data_ptr(),
                                                  _stream()), "moe_plan_wide")
        return
    _n.check(_n.cuda_lib().cafd_moe_plan(idx.data_ptr(), T, k, E, tile_rows, C.byref(layout), dest_row.data_ptr(),
                                         _ptr(expert_count), status_word(idx.device).data_ptr(), _stream()), "moe_plan")


WIDE_PLAN_ENTRIES = 8192      # (token, slot) entries from which the plan runs in its three-launch wide form
_plan_scratch: dict = {}


_route_scratch: dict = {}


def norm_route(h: torch.Tensor, ln_w: torch.Tensor, eps: float, router_w: torch.Tensor, x_out: torch.Tensor, out_idx: torch.Tensor,
               out_w: torch.Tensor, top_k: int, *, scoring: str = "softmax", bias: torch.Tensor | None = None, num_groups: int = 1,
               topk_groups: int = 1, normalize: bool = True, routed_scale: float = 1.0,
               logits_out: torch.Tensor | None = None) -> None:
    """x_out = RMSNorm(h) * ln_w, router scores x_out @ router_w.T and the top-k routing of every row in one launch
    (grid token x 8 expert groups; meant for decode-sized batches).  ``logits_out`` [T, E] fp32 receives the scores
    (a per-device scratch is used when it is not given)."""
    T, H = h.shape
    E = router_w.shape[0]
    key = h.device.index
    sc = _route_scratch.get(key)
    if sc is None or sc[0].shape[0] < T or sc[0].shape[1] < E:
        sc = (torch.empty(max(T, 256), max(E, 512), dtype=torch.float32, device=h.device),
              torch.zeros(max(T, 256), dtype=torch.int32, device=h.device))
        _route_scratch[key] = sc
    buf = logits_out if logits_out is not None else sc[0].view(-1)[:T * E].view(T, E)
    assert buf.is_contiguous()
    _n.check(_n.cuda_lib().cafd_norm_route(h.data_ptr(), ln_w.data_ptr(), eps, router_w.data_ptr(), _ptr(bias), x_out.data_ptr(),
                                           out_idx.data_ptr(), out_w.data_ptr(), buf.data_ptr(), sc[1].data_ptr(), T, H, E, top_k,
                                           int(scoring == "sigmoid"), num_groups, topk_groups, int(normalize), routed_scale,
                                           _stream()), "norm_route")


def moe_dispatch(x: torch.Tensor, idx: torch.Tensor, dest_row: torch.Tensor, layout: "_n.MoeLayout",
                 epoch: torch.Tensor, done_counter: torch.Tensor) -> None:
    T, k = idx.shape
    _n.check(_n.cuda_lib().cafd_moe_dispatch(x.data_ptr(), idx.data_ptr(), dest_row.data_ptr(), T, k, x.shape[1],
                                             C.byref(layout), epoch.data_ptr(), done_counter.data_ptr(), _stream()),
             "moe_dispatch")


def moe_combine(buf: torch.Tensor, w: torch.Tensor, out: torch.Tensor, *, shared: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, flags_ptr: int | None = None, n_flags: int = 0,
                epoch: torch.Tensor | None = None, norm_w: torch.Tensor | None = None, eps: float = 0.0,
                x_out: torch.Tensor | None = None) -> torch.Tensor:
    """out = sum_s w[t, s] * buf[t, s] + shared + residual (one rounding); with ``norm_w`` also
    x_out = RMSNorm(out) * norm_w (the next layer's input norm) in the same launch."""
    T, k = w.shape
    H = out.shape[1]
    if norm_w is not None and H <= 8192:
        _n.check(_n.cuda_lib().cafd_moe_combine_norm(buf.data_ptr(), w.data_ptr(), _ptr(shared), _ptr(residual), out.data_ptr(),
                                                     T, k, H, flags_ptr, n_flags, _ptr(epoch), status_word(out.device).data_ptr(),
                                                     norm_w.data_ptr(), eps, x_out.data_ptr(), _stream()), "moe_combine_norm")
        return out
    _n.check(_n.cuda_lib().cafd_moe_combine(buf.data_ptr(), w.data_ptr(), _ptr(shared), _ptr(residual), out.data_ptr(),
                                            T, k, H, flags_ptr, n_flags, _ptr(epoch),
                                            status_word(out.device).data_ptr(), _stream()), "moe_combine")
    if norm_w is not None:
        rmsnorm(out, norm_w, eps, out=x_out)
    return out


# ---- attention -------------------------------------------------------------------------------------
def attn_decode_splits(num_seqs: int, tiles_per_seq: int, Hkv: int, max_pages: int, window: int = 0) -> int:
    """KV splits for the decode attention kernel (``window`` > 0: a row reads at most the pages its window touches, so
    the splits are sized for those, not for the whole table).  The kernel keeps one 64-token page pair in flight per CTA, so
    HBM is only saturated with about three CTAs per SM (64 KB of shared memory each): aim for one full wave of
    3 x SMs CTAs, and never let a split grow past ~1K tokens (measured: 8 x 8K context 46 -> 33 us, 32 x 8K
    131 -> 99 us against the old one-CTA-per-SM rule)."""
    if window > 0:
        max_pages = min(max_pages, (window + 63) // 64 + 1)
    ctas = max(1, num_seqs * tiles_per_seq * Hkv)
    want = max((3 * num_sms()) // ctas, (max_pages + 15) // 16, 1)
    return max(1, min(want, max(1, max_pages // 4), 32))


def set_fixed_kv_split(tokens: int) -> None:
    """Batch-invariant decode attention: > 0 makes every kv split of the decode kernels (GQA and dense MLA) cover
    ``tokens`` positions (a multiple of 64) counted from position 0, so that a row's partial sums and their merge order
    depend on its own length only; callers then launch ``kv_splits(max_pages)`` splits.  0 restores the even division
    that fills the GPU.  Counterpart of the reference's fixed (warps, groups) K-walk at every decode width
    (REPORT-kernel-210.md:14-66)."""
    _n.check(_n.cuda_lib().cafd_set_fixed_kv_split(int(tokens)), "set_fixed_kv_split")


def fixed_kv_split() -> int:
    return int(_n.cuda_lib().cafd_fixed_kv_split())


BATCH_INVARIANT_SPLIT = 1024     # tokens per kv split when CAFD_BATCH_INVARIANT=1 asks for the mode


def batch_invariant_from_env() -> int:
    """Engines call this once when they are built: ``CAFD_BATCH_INVARIANT=1`` switches the library to fixed kv splits
    (unless a split size was set by hand) and returns the split size; without it the current setting is returned."""
    import os
    if os.environ.get("CAFD_BATCH_INVARIANT", "0") == "1" and fixed_kv_split() == 0:
        set_fixed_kv_split(BATCH_INVARIANT_SPLIT)
    return fixed_kv_split()


def kv_splits_fixed(max_pages: int, cap: int = 0) -> int:
    """Splits to launch in the fixed-split mode: enough to cover the widest row of the page table.  ``cap`` > 0: the
    kernel's limit on the number of splits (the mode is refused when the table is wider than cap x split)."""
    n = max(1, -(-max_pages * 64 // fixed_kv_split()))
    if cap and n > cap:
        raise ValueError(f"a page table of {max_pages} pages needs {n} kv splits of {fixed_kv_split()} tokens, the kernel takes {cap}")
    return n


def attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                seq_lens: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor, scratch: torch.Tensor | None,
                max_q_len: int, splits: int, scale: float | None = None, window: int = 0) -> torch.Tensor:
    """``window`` > 0: a query at position t sees keys (t - window, t] only (sliding-window layers); the pages
    before the window are not read."""
    _, Hq, D = q.shape
    Hkv = k_cache.shape[1]                 # pools are [pages, kv heads, 64, D]
    num_seqs, max_pages = page_table.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    _n.check(_n.cuda_lib().cafd_attn_decode(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(),
                                            seq_lens.data_ptr(), q_start.data_ptr(), out.data_ptr(), _ptr(scratch),
                                            num_seqs, max_q_len, max_pages, Hq, Hkv, D, splits, scale, int(window), _stream()),
             "attn_decode")
    return out


def attn_decode_partial(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                        seq_lens: torch.Tensor, kv_base: torch.Tensor, q_start: torch.Tensor, peer_scratch: list[int], my_rank: int,
                        max_q_len: int, splits: int, scale: float | None = None) -> None:
    """Context split, first half: attention over the pages this rank holds; the unnormalised partials (O, m, l) go into
    every rank's scratch (``peer_scratch`` device addresses, this rank's own included) at this rank's split slots."""
    _, Hq, D = q.shape
    Hkv = k_cache.shape[1]
    num_seqs, max_pages = page_table.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    arr = (C.c_void_p * 8)(*peer_scratch)
    _n.check(_n.cuda_lib().cafd_attn_decode_partial(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(),
                                                    seq_lens.data_ptr(), kv_base.data_ptr(), q_start.data_ptr(), arr, len(peer_scratch),
                                                    my_rank, num_seqs, max_q_len, max_pages, Hq, Hkv, D, splits, scale, _stream()),
             "attn_decode_partial")


def attn_merge(scratch: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor, max_q_len: int, Hkv: int, total_splits: int) -> torch.Tensor:
    """Context split, second half: merge ``total_splits`` partials per (tile, kv head) in slot order into ``out``
    [total_q, Hq, D]."""
    _, Hq, _ = out.shape
    _n.check(_n.cuda_lib().cafd_attn_merge(scratch.data_ptr(), q_start.data_ptr(), out.data_ptr(), q_start.shape[0] - 1, max_q_len,
                                           Hq, Hkv, total_splits, _stream()), "attn_merge")
    return out


def attn_decode_scratch_floats(num_seqs: int, max_q_len: int, Hq: int, Hkv: int, splits: int) -> int:
    q_per_tile = 16 // (Hq // Hkv)
    tiles = (max_q_len + q_per_tile - 1) // q_per_tile
    return int(_n.cuda_lib().cafd_attn_decode_scratch_floats(num_seqs, tiles, Hkv, splits))


def attn_prefill(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, page_table: torch.Tensor,
                 seq_lens: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor, max_q_len: int,
                 scale: float | None = None, window: int = 0) -> torch.Tensor:
    total_q, Hq, D = q.shape
    num_pages, Hkv, _, _ = k_cache.shape   # pools are [pages, kv heads, 64, D]
    num_seqs, max_pages = page_table.shape
    scale = scale if scale is not None else 1.0 / math.sqrt(D)
    _n.check(_n.cuda_lib().cafd_attn_prefill(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), page_table.data_ptr(),
                                             seq_lens.data_ptr(), q_start.data_ptr(), out.data_ptr(),
                                             status_word(q.device).data_ptr(), total_q, num_seqs, max_q_len, num_pages,
                                             max_pages, Hq, Hkv, D, scale, int(window), _stream()), "attn_prefill")
    return out


def mla_blocks(q_lens: list[int], heads: int) -> tuple[list[int], list[int]]:
    """Row-block table for ``mla_attention``: every block covers 128 / heads query tokens of one sequence."""
    per = 128 // heads
    seqs, toks = [], []
    for s, n in enumerate(q_lens):
        for t0 in range(0, n, per):
            seqs.append(s)
            toks.append(t0)
    return seqs, toks


def mla_scratch_floats(n_blocks: int, splits: int) -> int:
    return int(_n.cuda_lib().cafd_mla_scratch_floats(n_blocks, splits))


def mla_attention(q_abs: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor, seq_lens: torch.Tensor,
                  q_start: torch.Tensor, block_seq: torch.Tensor, block_tok0: torch.Tensor, out: torch.Tensor,
                  scale: float, splits: int = 1, scratch: torch.Tensor | None = None, out_tpad: int = 0,
                  sparse_idx: torch.Tensor | None = None, gathered: torch.Tensor | None = None) -> torch.Tensor:
    """Absorbed MLA: q_abs [tokens, heads, 576] (512 latent-projected + 64 rope), cache [pages, 64, 576]
    (page 0 zero), out [tokens, heads, 512] = softmax(q c^T * scale) c[:, :512] with the causal rule
    that query token i of a sequence sees kv positions <= seq_len - q_len + i.  With ``out_tpad`` > 0
    the output is head-major: out [heads, out_tpad, 512].  With ``sparse_idx`` [tokens, k] (ascending positions,
    -1 padded; from ``index_topk``) each block must be a single token (``mla_blocks(q_lens, 128)``) and the
    token attends to its listed positions only.  With ``gathered`` [blocks, k, 576] (from ``mla_fp8_gather``) the
    listed records are read from that buffer instead of the cache, which may then be None."""
    T, heads, rec = q_abs.shape
    assert rec == 576 and 128 % heads == 0 and q_abs.is_contiguous() and out.is_contiguous()
    _, max_pages = page_table.shape
    if gathered is not None:
        k = sparse_idx.shape[1]
        assert gathered.dtype == torch.bfloat16 and gathered.is_contiguous() and gathered.numel() >= max(block_seq.numel() * k, 64) * 576
        _n.check(_n.cuda_lib().cafd_mla_attention_gathered(
            q_abs.data_ptr(), gathered.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), q_start.data_ptr(),
            block_seq.data_ptr(), block_tok0.data_ptr(), out.data_ptr(), _ptr(scratch), status_word(q_abs.device).data_ptr(),
            T * heads, block_seq.numel(), max_pages, heads, splits, out_tpad, scale, sparse_idx.data_ptr(), k, _stream()),
            "mla_attention_gathered")
        return out
    assert cache.is_contiguous() and cache.dtype == torch.bfloat16
    num_pages = cache.shape[0]
    _n.check(_n.cuda_lib().cafd_mla_attention(q_abs.data_ptr(), cache.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(),
                                              q_start.data_ptr(), block_seq.data_ptr(), block_tok0.data_ptr(), out.data_ptr(),
                                              _ptr(scratch), status_word(q_abs.device).data_ptr(), T * heads,
                                              block_seq.numel(), num_pages, max_pages, heads, splits, out_tpad, scale,
                                              _ptr(sparse_idx), sparse_idx.shape[1] if sparse_idx is not None else 0, _stream()),
             "mla_attention")
    return out


def mla_attention_partial(q_abs: torch.Tensor, cache: torch.Tensor, page_table: torch.Tensor, seq_lens: torch.Tensor,
                          kv_base: torch.Tensor, q_start: torch.Tensor, block_seq: torch.Tensor, block_tok0: torch.Tensor,
                          peer_scratch: list[int], my_rank: int, scale: float, splits: int) -> None:
    """Context split, first half (absorbed MLA): attention over the records this rank holds (``seq_lens`` local lengths,
    ``kv_base`` visibility bases); the unnormalised partials go into every rank's scratch (``peer_scratch`` device
    addresses, this rank's own included) at this rank's split slots."""
    T, heads, rec = q_abs.shape
    assert rec == 576 and 128 % heads == 0 and q_abs.is_contiguous() and cache.is_contiguous() and cache.dtype == torch.bfloat16
    arr = (C.c_void_p * 8)(*peer_scratch)
    _n.check(_n.cuda_lib().cafd_mla_attention_partial(
        q_abs.data_ptr(), cache.data_ptr(), page_table.data_ptr(), seq_lens.data_ptr(), kv_base.data_ptr(), q_start.data_ptr(),
        block_seq.data_ptr(), block_tok0.data_ptr(), arr, len(peer_scratch), my_rank, status_word(q_abs.device).data_ptr(),
        T * heads, block_seq.numel(), cache.shape[0], page_table.shape[1], heads, splits, scale, _stream()), "mla_attention_partial")


def mla_merge(scratch: torch.Tensor, block_seq: torch.Tensor, block_tok0: torch.Tensor, q_start: torch.Tensor, out: torch.Tensor,
              heads: int, total_splits: int, out_tpad: int = 0) -> torch.Tensor:
    """Context split, second half: merge ``total_splits`` partials per (row block, output half) in slot order."""
    _n.check(_n.cuda_lib().cafd_mla_merge(scratch.data_ptr(), block_seq.data_ptr(), block_tok0.data_ptr(), q_start.data_ptr(),
                                          out.data_ptr(), block_seq.numel(), heads, total_splits, out_tpad, _stream()), "mla_merge")
    return out


FP8_RECORD_BYTES = 656      # 512 E4M3 latents + 4 fp32 scales + 64 bf16 rope dims


def mla_fp8_gather(cache: torch.Tensor, sparse_idx: torch.Tensor, page_table: torch.Tensor, seq_lens: torch.Tensor,
                   q_start: torch.Tensor, block_seq: torch.Tensor, block_tok0: torch.Tensor, out: torch.Tensor) -> torch.Tensor:
    """Expand the FP8 records [pages, 64, 656] (uint8) that ``sparse_idx`` [tokens, k] lists into out [blocks, k, 576]
    bf16; one block per query token, as in sparse attention.  Entries that do not exist are left untouched."""
    assert cache.dtype == torch.uint8 and cache.shape[-1] == FP8_RECORD_BYTES and cache.is_contiguous()
    k = sparse_idx.shape[1]
    assert out.dtype == torch.bfloat16 and out.is_contiguous() and out.numel() >= block_seq.numel() * k * 576
    _n.check(_n.cuda_lib().cafd_mla_fp8_gather(cache.data_ptr(), sparse_idx.data_ptr(), k, page_table.data_ptr(),
                                               page_table.shape[1], seq_lens.data_ptr(), q_start.data_ptr(),
                                               block_seq.data_ptr(), block_tok0.data_ptr(), block_seq.numel(), out.data_ptr(),
                                               _stream()), "mla_fp8_gather")
    return out


def indexer_scores(q_idx: torch.Tensor, k_cache: torch.Tensor, head_w: torch.Tensor, page_table: torch.Tensor,
                   seq_lens: torch.Tensor, q_start: torch.Tensor, block_seq: torch.Tensor, block_tok0: torch.Tensor,
                   scores: torch.Tensor, splits: int = 1, w_scale: float = 1.0) -> torch.Tensor:
    """scores[t, s] = sum_h w_scale * head_w[t, h] * relu(q_idx[t, h] . k_cache[s]) for visible s, -inf beyond (inside
    the 128-position tiles that were computed).  q_idx [T, heads, 128] bf16; head_w [T, heads] bf16 (any row stride);
    k_cache [pages, 64, 128] bf16; blocks cover 256 / heads tokens (``mla_blocks(q_lens, heads // 2)``)."""
    T, heads, d = q_idx.shape
    assert d == 128 and q_idx.is_contiguous() and head_w.dtype == torch.bfloat16 and head_w.stride(1) == 1
    assert scores.dtype == torch.float32 and scores.stride(1) == 1
    _n.check(_n.cuda_lib().cafd_indexer_scores(q_idx.data_ptr(), k_cache.data_ptr(), head_w.data_ptr(), head_w.stride(0), w_scale,
                                               page_table.data_ptr(), seq_lens.data_ptr(), q_start.data_ptr(),
                                               block_seq.data_ptr(), block_tok0.data_ptr(), scores.data_ptr(),
                                               status_word(q_idx.device).data_ptr(), T * heads, block_seq.numel(),
                                               k_cache.shape[0], page_table.shape[1], heads, splits, scores.stride(0),
                                               _stream()), "indexer_scores")
    return scores


def index_topk(scores: torch.Tensor, top_k: int, out: torch.Tensor, limits: torch.Tensor | None = None,
               seq_lens: torch.Tensor | None = None, q_start: torch.Tensor | None = None) -> torch.Tensor:
    """Top ``top_k`` positions per row among the visible scores: ties to the lower position, ascending output, -1
    padded.  The visible count is ``limits[t]``, or derived from (seq_lens, q_start) like the attention kernels do."""
    T = scores.shape[0]
    assert out.shape == (T, top_k) and out.dtype == torch.int32 and out.is_contiguous()
    S = q_start.numel() - 1 if q_start is not None else 0
    _n.check(_n.cuda_lib().cafd_index_topk(scores.data_ptr(), scores.stride(0), _ptr(limits), _ptr(seq_lens), _ptr(q_start), S,
                                           T, top_k, out.data_ptr(), _stream()), "index_topk")
    return out


def index_k_store(k: torch.Tensor, slots: torch.Tensor, cache: torch.Tensor) -> None:
    _n.check(_n.cuda_lib().cafd_index_k_store(k.data_ptr(), k.stride(0), slots.data_ptr(), cache.data_ptr(), k.shape[0],
                                              _stream()), "index_k_store")


def mla_prep_a(a: torch.Tensor, q_lora: int, q_norm_w: torch.Tensor | None, kv_norm_w: torch.Tensor, inv_freq: torch.Tensor,
               positions: torch.Tensor, slots: torch.Tensor, q_a_out: torch.Tensor | None, cache: torch.Tensor, eps: float,
               interleaved: bool, lat_out: torch.Tensor | None = None) -> None:
    """a [T, q_lora + 576] -> q_a_out [T, q_lora] (normalised) and the [latent | rope] record at cache slot ``slots[t]``.
    A bf16 cache [.., 576] takes bf16 records; a uint8 cache [.., 656] takes FP8 records (E4M3 latents with one fp32
    scale per 128, bf16 rope)."""
    T = a.shape[0]
    assert a.shape[1] == q_lora + 576 and a.stride(1) == 1
    fp8 = cache.dtype == torch.uint8
    assert cache.shape[-1] == (FP8_RECORD_BYTES if fp8 else 576) and (fp8 or cache.dtype == torch.bfloat16)
    fn = _n.cuda_lib().cafd_mla_prep_a_fp8 if fp8 else _n.cuda_lib().cafd_mla_prep_a
    _n.check(fn(a.data_ptr(), a.stride(0), q_lora, _ptr(q_norm_w), kv_norm_w.data_ptr(), inv_freq.data_ptr(),
                positions.data_ptr(), slots.data_ptr(), _ptr(q_a_out), cache.data_ptr(), T, eps, int(interleaved),
                _ptr(lat_out), _stream()), "mla_prep_a")


def attn_prefill_mla(q_nope: torch.Tensor, q_rope: torch.Tensor, k_exp: torch.Tensor, v_exp: torch.Tensor, kv_tmp_start: torch.Tensor,
                     latent_cache: torch.Tensor, page_table: torch.Tensor, seq_lens: torch.Tensor, q_start: torch.Tensor,
                     out: torch.Tensor, max_q_len: int, heads: int, scale: float, qr_col0: int = 512) -> torch.Tensor:
    """MLA prefill in expanded form.  q_nope [T, heads * 192] (first 128 columns of each head are used), q_rope
    [T, heads, 576]-like buffer holding the rotated rope dims at ``qr_col0`` of every head, k_exp / v_exp
    [rows, heads * 128] (kv_b applied to the cached latents in order; rows a multiple of 64), the latent cache for
    the shared rope keys.  out [T, heads, 128]."""
    T = q_nope.shape[0]
    S, max_pages = page_table.shape
    qs, qrs = q_nope.shape[1] // heads, q_rope.numel() // (q_rope.shape[0] * heads)
    assert k_exp.shape[0] % 64 == 0 and k_exp.shape[1] == heads * 128 and k_exp.is_contiguous() and v_exp.is_contiguous()
    _n.check(_n.cuda_lib().cafd_attn_prefill_mla(q_nope.data_ptr(), qs, q_rope.data_ptr(), qrs, qr_col0, k_exp.data_ptr(),
                                                 v_exp.data_ptr(), k_exp.shape[0], kv_tmp_start.data_ptr(), latent_cache.data_ptr(),
                                                 page_table.data_ptr(), seq_lens.data_ptr(), q_start.data_ptr(), out.data_ptr(),
                                                 status_word(q_nope.device).data_ptr(), T, S, max_q_len, latent_cache.shape[0],
                                                 max_pages, heads, scale, _stream()), "attn_prefill_mla")
    return out


def mla_q_split(q: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor, slab: torch.Tensor, q_abs: torch.Tensor,
                heads: int, interleaved: bool) -> None:
    """q [T, heads*192] -> slab [heads, t_pad, 128] (nope dims, head-major) and q_abs[:, :, 512:] (rotated rope dims)."""
    T = q.shape[0]
    assert q.shape[1] == heads * 192 and slab.shape[0] == heads and slab.shape[2] == 128
    _n.check(_n.cuda_lib().cafd_mla_q_split(q.data_ptr(), q.stride(0), inv_freq.data_ptr(), positions.data_ptr(),
                                            slab.data_ptr(), q_abs.data_ptr(), T, heads, slab.shape[1], int(interleaved),
                                            _stream()), "mla_q_split")


MLA_SMALL_ROWS = 16      # steps of at most this many rows take the decode-sized absorb / un-absorb kernels


def mla_absorb_small(q: torch.Tensor, w_uk: torch.Tensor, inv_freq: torch.Tensor, positions: torch.Tensor, q_abs: torch.Tensor,
                     heads: int, interleaved: bool) -> None:
    """Decode-sized steps (T <= 16): q [T, heads*192] -> q_abs [T, heads, 576] in one launch: the 128 nope dims of
    every head multiplied by W_uk[h] [512, 128] into the latent part, the 64 rope dims rotated into the tail."""
    T = q.shape[0]
    assert T <= MLA_SMALL_ROWS and q.shape[1] == heads * 192 and w_uk.shape == (heads, 512, 128) and w_uk.is_contiguous()
    _n.check(_n.cuda_lib().cafd_mla_absorb_small(q.data_ptr(), q.stride(0), w_uk.data_ptr(), inv_freq.data_ptr(),
                                                 positions.data_ptr(), q_abs.data_ptr(), T, heads, int(interleaved), _stream()),
             "mla_absorb_small")


def mla_unabsorb_small(o_lat: torch.Tensor, w_uv: torch.Tensor, attn: torch.Tensor, T: int) -> None:
    """Decode-sized steps: o_lat [heads, t_pad, 512] (head-major attention output) -> attn [T, heads*128] through
    W_uv[h] [128, 512]."""
    heads, t_pad, _ = o_lat.shape
    assert T <= MLA_SMALL_ROWS and w_uv.shape == (heads, 128, 512) and w_uv.is_contiguous() and attn.is_contiguous()
    _n.check(_n.cuda_lib().cafd_mla_unabsorb_small(o_lat.data_ptr(), t_pad, w_uv.data_ptr(), attn.data_ptr(), T, heads, _stream()),
             "mla_unabsorb_small")


# ---- sampling ---------------------------------------------------------------------------------------------
_SAMPLE_ROW = None


def sample_row_dtype():
    """numpy dtype of the 64-byte row record read by the sampling kernel."""
    global _SAMPLE_ROW
    if _SAMPLE_ROW is None:
        import numpy as np
        _SAMPLE_ROW = np.dtype([("temperature", "<f4"), ("top_p", "<f4"), ("min_p", "<f4"), ("top_k", "<i4"), ("seed", "<u8"),
                                ("position", "<i8"), ("mask_word0", "<i8"), ("logits_row", "<i4"), ("pad", "<i4", (5,))])
        assert _SAMPLE_ROW.itemsize == 64
    return _SAMPLE_ROW


def pack_sample_rows(params, positions, logits_rows=None, mask_word0=None) -> torch.Tensor:
    """Host-side row records (uint8 tensor [n, 64]) for ``sample_rows`` from SamplingParams-like objects."""
    import numpy as np
    n = len(params)
    rec = np.zeros(n, dtype=sample_row_dtype())
    for i, p in enumerate(params):
        rec[i]["temperature"], rec[i]["top_p"], rec[i]["min_p"] = p.temperature, p.top_p, p.min_p
        rec[i]["top_k"] = p.top_k if p.top_k is not None else 0
        rec[i]["seed"], rec[i]["position"] = p.seed & 0xFFFFFFFFFFFFFFFF, positions[i]
        rec[i]["mask_word0"] = -1 if mask_word0 is None or mask_word0[i] is None else mask_word0[i]
        rec[i]["logits_row"] = i if logits_rows is None else logits_rows[i]
    return torch.from_numpy(rec.view(np.uint8).reshape(n, 64))


def sample_rows(logits: torch.Tensor, rows: torch.Tensor, out_token: torch.Tensor, out_status: torch.Tensor,
                masks: torch.Tensor | None = None) -> None:
    """Exact target sampling: ``rows`` is a device uint8 [n, 64] tensor of row records, ``masks`` packed int32 bits."""
    assert logits.dtype == torch.float32 and logits.stride(1) == 1 and rows.dtype == torch.uint8 and rows.shape[1] == 64
    _n.check(_n.cuda_lib().cafd_sample_rows(logits.data_ptr(), logits.stride(0), logits.shape[1], rows.data_ptr(), _ptr(masks),
                                            rows.shape[0], out_token.data_ptr(), out_status.data_ptr(), _stream()), "sample_rows")


def accept_prefix(selected: torch.Tensor, draft: torch.Tensor, row_start: torch.Tensor, accepted: torch.Tensor,
                  bonus: torch.Tensor) -> None:
    S = row_start.numel() - 1
    _n.check(_n.cuda_lib().cafd_accept_prefix(selected.data_ptr(), draft.data_ptr(), row_start.data_ptr(), S,
                                              accepted.data_ptr(), bonus.data_ptr(), _stream()), "accept_prefix")


# ---- FP8 block-scaled GEMM -----------------------------------------------------------------------------
def quant_rows_fp8(x: torch.Tensor, q: torch.Tensor | None = None, s: torch.Tensor | None = None):
    """bf16 [T, K] -> (E4M3 [T, K], fp32 scales [T, K/128]); scale = amax/448 per row and 128 columns."""
    T, Kd = x.shape
    assert x.dtype == torch.bfloat16 and x.stride(1) == 1 and Kd % 128 == 0
    if q is None:
        q = torch.empty(T, Kd, dtype=torch.float8_e4m3fn, device=x.device)
    if s is None:
        s = torch.empty(T, Kd // 128, dtype=torch.float32, device=x.device)
    _n.check(_n.cuda_lib().cafd_quant_rows_fp8(x.data_ptr(), q.data_ptr(), s.data_ptr(), T, Kd, x.stride(0), _stream()),
             "quant_rows_fp8")
    return q, s


def _fp8_common(a: "_n.GemmArgs", device: torch.device, split_k: bool) -> None:
    a.status = status_word(device).data_ptr()
    a.out_f32, a.fp8, a.num_sms = 0, 1, num_sms()
    if a.swap and split_k:
        _attach_splitk(a, device)


def linear_fp8(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out: torch.Tensor | None = None, *,
               w_up: torch.Tensor | None = None, ws_up: torch.Tensor | None = None, residual: torch.Tensor | None = None,
               swap: bool | None = None, split_k: bool = True) -> torch.Tensor:
    """y = dequant(xq, xs) @ dequant(wq, ws).T with E4M3 operands on the tensor cores.

    xq [T, K] e4m3 + xs [T, K/128]; wq [N, K] e4m3 + ws [N/128, K/128].  ``w_up``: SwiGLU pair."""
    T, Kd = xq.shape
    N = wq.shape[0]
    assert xq.is_contiguous() and wq.is_contiguous() and xs.is_contiguous() and ws.is_contiguous() and N % 128 == 0
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=xq.device)
    if T == 0:
        return out
    if swap is None:
        swap = T <= 64
    a = _n.GemmArgs()
    a.w0, a.w1, a.x, a.out = wq.data_ptr(), _ptr(w_up), xq.data_ptr(), out.data_ptr()
    a.w_scale, a.w_scale1, a.x_scale = ws.data_ptr(), _ptr(ws_up), xs.data_ptr()
    a.residual = _ptr(residual)
    a.w_rows_total, a.x_rows_total = N, T
    a.k, a.n_features, a.x_rows, a.ldo = Kd, N, T, out.stride(0)
    a.w_rows_per_expert, a.w1_row_offset, a.max_x_tiles = 0, 0, 0
    a.swap, a.dual = int(swap), int(w_up is not None)
    a.bx = (64 if (w_up is not None and T > 32) else pick_token_tile(T)) if swap else 128
    if swap and T > a.bx:
        a.bx = 64 if w_up is not None else 128
    _fp8_common(a, xq.device, split_k)
    _n.check(_n.cuda_lib().cafd_gemm_fp8(C.byref(a), _stream()), "cafd_gemm_fp8")
    return out


def grouped_linear_fp8(xq: torch.Tensor, xs: torch.Tensor, wq: torch.Tensor, ws: torch.Tensor, out: torch.Tensor,
                       tile_expert: torch.Tensor, tile_row0: torch.Tensor, num_tiles: torch.Tensor, max_tiles: int,
                       tile_rows: int, *, w_up: torch.Tensor | None = None, ws_up: torch.Tensor | None = None,
                       row_dst: torch.Tensor | None = None, wait_flag: int | None = None, epoch: torch.Tensor | None = None,
                       signal_flag: int | None = None, done_counter: torch.Tensor | None = None, out_ptr: int | None = None,
                       ldo: int | None = None, split_k: bool = True) -> None:
    """Expert-grouped FP8 GEMM over an expert-sorted E4M3 slab (wq [E, N, K], ws [E, N/128, K/128])."""
    E, N, Kd = wq.shape
    a = _n.GemmArgs()
    a.w0, a.w1, a.x = wq.data_ptr(), _ptr(w_up), xq.data_ptr()
    a.w_scale, a.w_scale1, a.x_scale = ws.data_ptr(), _ptr(ws_up), xs.data_ptr()
    a.out = out_ptr if out_ptr is not None else out.data_ptr()
    a.row_dst = _ptr(row_dst)
    a.tile_expert, a.tile_row0, a.num_x_tiles = tile_expert.data_ptr(), tile_row0.data_ptr(), num_tiles.data_ptr()
    a.wait_flag, a.epoch = wait_flag, _ptr(epoch)
    a.signal_flag, a.done_counter = signal_flag, _ptr(done_counter)
    a.w_rows_total, a.x_rows_total = E * N, xq.shape[0]
    a.k, a.n_features, a.x_rows = Kd, N, xq.shape[0]
    a.ldo = ldo if ldo is not None else out.stride(0)
    a.w_rows_per_expert, a.w1_row_offset, a.max_x_tiles = N, 0, max_tiles
    a.swap, a.dual, a.bx = int(tile_rows < 128), int(w_up is not None), tile_rows
    _fp8_common(a, xq.device, split_k)
    _n.check(_n.cuda_lib().cafd_gemm_fp8(C.byref(a), _stream()), "cafd_gemm_fp8(grouped)")


# ---- 4-bit weights (MXFP4 / NVFP4) --------------------------------------------------------------------------
W4_FORMATS = {"mxfp4": 2, "nvfp4": 3}


def linear_w4(x: torch.Tensor, w: tuple, fmt: str, out: torch.Tensor | None = None, *, w_up: tuple | None = None,
              residual: torch.Tensor | None = None, out_f32: bool = False) -> torch.Tensor:
    """y = x @ dequant(w).T for T <= 128 rows with the weights expanded on the way into shared memory.
    ``w`` = (packed [N, K/2] uint8, block scales [N, K/32] UE8M0 or [N, K/16] E4M3, global fp32 [1] or None);
    ``w_up`` selects SwiGLU.  Larger batches: ``w4_dequant`` + ``linear``."""
    T, Kd = x.shape
    packed, scales, glob = w
    N = packed.shape[0]
    assert T <= 128 and Kd % 128 == 0 and packed.shape[1] * 2 == Kd and x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        out = torch.empty(T, N, dtype=torch.float32 if out_f32 else torch.bfloat16, device=x.device)
    a = _n.GemmArgs()
    a.w0, a.w1, a.x, a.out = packed.data_ptr(), (w_up[0].data_ptr() if w_up else None), x.data_ptr(), out.data_ptr()
    a.w_scale, a.w_scale1 = scales.data_ptr(), (w_up[1].data_ptr() if w_up else None)
    a.residual = _ptr(residual)
    a.status = status_word(x.device).data_ptr()
    a.w_rows_total, a.x_rows_total = N, T
    a.k, a.n_features, a.x_rows, a.ldo = Kd, N, T, out.stride(0)
    a.w_rows_per_expert = N
    a.swap, a.dual, a.bx = 1, int(w_up is not None), pick_token_tile(T)
    a.out_f32, a.num_sms = int(out_f32), num_sms()
    _n.check(_n.cuda_lib().cafd_gemm_w4(C.byref(a), W4_FORMATS[fmt], _ptr(glob), _ptr(w_up[2]) if w_up else None, _stream()),
             "cafd_gemm_w4")
    return out


def grouped_linear_w4(x: torch.Tensor, w: tuple, fmt: str, out: torch.Tensor, tile_expert: torch.Tensor, tile_row0: torch.Tensor,
                      num_tiles: torch.Tensor, max_tiles: int, tile_rows: int, *, w_up: tuple | None = None,
                      row_dst: torch.Tensor | None = None, wait_flag: int | None = None, epoch: torch.Tensor | None = None,
                      signal_flag: int | None = None, done_counter: torch.Tensor | None = None, out_ptr: int | None = None,
                      ldo: int | None = None) -> None:
    """Expert-grouped form: ``w`` = (packed [E, N, K/2], scales [E, N, K/g], global fp32 [E] or None); tile_rows <= 128
    (<= 64 with ``w_up``)."""
    packed, scales, glob = w
    E, N, Kh = packed.shape
    a = _n.GemmArgs()
    a.w0, a.w1, a.x = packed.data_ptr(), (w_up[0].data_ptr() if w_up else None), x.data_ptr()
    a.w_scale, a.w_scale1 = scales.data_ptr(), (w_up[1].data_ptr() if w_up else None)
    a.out = out_ptr if out_ptr is not None else out.data_ptr()
    a.row_dst = _ptr(row_dst)
    a.tile_expert, a.tile_row0, a.num_x_tiles = tile_expert.data_ptr(), tile_row0.data_ptr(), num_tiles.data_ptr()
    a.wait_flag, a.epoch = wait_flag, _ptr(epoch)
    a.signal_flag, a.done_counter = signal_flag, _ptr(done_counter)
    a.status = status_word(x.device).data_ptr()
    a.w_rows_total, a.x_rows_total = E * N, x.shape[0]
    a.k, a.n_features, a.x_rows = Kh * 2, N, x.shape[0]
    a.ldo = ldo if ldo is not None else out.stride(0)
    a.w_rows_per_expert, a.max_x_tiles = N, max_tiles
    a.swap, a.dual, a.bx = 1, int(w_up is not None), tile_rows
    a.num_sms = num_sms()
    _n.check(_n.cuda_lib().cafd_gemm_w4(C.byref(a), W4_FORMATS[fmt], _ptr(glob), _ptr(w_up[2]) if w_up else None, _stream()),
             "cafd_gemm_w4(grouped)")


def w4_dequant(w: tuple, fmt: str, out: torch.Tensor | None = None) -> torch.Tensor:
    """Packed 4-bit weights -> bf16 (same leading shape, last dim K); NVFP4 folds the global scale in."""
    packed, scales, glob = w
    Kd = packed.shape[-1] * 2
    rows = packed.numel() // packed.shape[-1]
    if out is None:
        out = torch.empty(*packed.shape[:-1], Kd, dtype=torch.bfloat16, device=packed.device)
    rpe = packed.shape[-2] if packed.dim() == 3 else rows
    _n.check(_n.cuda_lib().cafd_w4_dequant(packed.data_ptr(), scales.data_ptr(), _ptr(glob), out.data_ptr(), rows, Kd,
                                           W4_FORMATS[fmt], rpe, _stream()), "w4_dequant")
    return out


def fp8_dequant_block128(q: torch.Tensor, scales: torch.Tensor, out: torch.Tensor | None = None) -> torch.Tensor:
    """E4M3 weights [..., N, K] with 128x128 block scales [..., N/128, K/128] -> bf16 (stacked experts are treated as
    one tall matrix: N must be a multiple of 128)."""
    Kd = q.shape[-1]
    rows = q.numel() // Kd
    assert q.shape[-2] % 128 == 0 and Kd % 128 == 0 and q.is_contiguous() and scales.is_contiguous()
    if out is None:
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=q.device)
    _n.check(_n.cuda_lib().cafd_fp8_dequant_block128(q.data_ptr(), scales.data_ptr(), out.data_ptr(), rows, Kd, _stream()),
             "fp8_dequant_block128")
    return out


# ---- EXL3 (trellis-coded weights) ---------------------------------------------------------------------------
_exl3_scratch: dict = {}


def linear_exl3(x: torch.Tensor, trellis: torch.Tensor, suh: torch.Tensor, svh: torch.Tensor, out: torch.Tensor | None = None,
                residual: torch.Tensor | None = None) -> torch.Tensor:
    """y = x @ W for an EXL3 tensor: trellis int16 [K/16, N/16, 16 * bits], suh [K] / svh [N] fp16 sign-scale vectors;
    W = H128_K-rotated, trellis-decoded, H128_N-rotated (see ``quant.codecs.exl3_dequant``).  T <= 128 rows."""
    T, Kd = x.shape
    Kt, Nt, W = trellis.shape
    N, bits = Nt * 16, W // 16
    assert Kt * 16 == Kd and Kd % 128 == 0 and N % 128 == 0 and T <= 128 and trellis.dtype == torch.int16 and trellis.is_contiguous()
    assert suh.dtype == torch.float16 and svh.dtype == torch.float16 and x.dtype == torch.bfloat16 and x.stride(1) == 1
    if out is None:
        out = torch.empty(T, N, dtype=torch.bfloat16, device=x.device)
    key = (x.device.index, Kd, N)
    sc = _exl3_scratch.get(key)
    if sc is None:
        sc = (torch.empty(128, Kd, dtype=torch.float16, device=x.device), torch.empty(128, N, dtype=torch.float32, device=x.device))
        _exl3_scratch[key] = sc
    _n.check(_n.cuda_lib().cafd_gemm_exl3(x.data_ptr(), x.stride(0), trellis.data_ptr(), suh.data_ptr(), svh.data_ptr(),
                                          _ptr(residual), out.data_ptr(), out.stride(0), sc[0].data_ptr(), sc[1].data_ptr(),
                                          status_word(x.device).data_ptr(), T, Kd, N, bits, pick_token_tile(T), num_sms(),
                                          _stream()), "cafd_gemm_exl3")
    return out
