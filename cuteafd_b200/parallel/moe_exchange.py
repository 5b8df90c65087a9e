"""Attention-rank / expert-rank halves of the MoE exchange.

Experts are partitioned by id over the expert ranks (``expert_range``).  The attention rank plans
the routes, stores token rows straight into each owner's slab (peer memory when the owner is
another GPU) and publishes a step number; the owner's grouped GEMMs wait for that number, run
fc1+SwiGLU and fc2, and the fc2 epilogue stores each (token, slot) row straight into the attention
rank's combine buffer and publishes the step number back.  With one GPU every pointer is local
and the same kernels run in stream order.

The reference moves the same data with a host transport worker and RoCE SEND/RECV
(rust/crates/cuteafd-daemon/src/shared/spark_waves.rs:1-84, 1188-1517) and sums TP slices
(rust/crates/cuteafd-transport/src/expert/topology.rs:1-7); expert-parallel dispatch/combine in
one kernel per direction is this engine's departure from it.
"""
from __future__ import annotations

from dataclasses import dataclass

import torch

from .._native import lib as _n
from ..ops import kernels as K
from ..ref.split import expert_range


def pick_tile_rows(T: int, top_k: int, num_experts: int) -> int:
    avg = T * top_k / max(1, num_experts)
    if avg <= 8:
        return 16
    if avg <= 24:
        return 32
    if avg <= 48:
        return 64
    return 128


def plan_tile_rows(fmt: str, T: int, top_k: int, num_experts: int) -> int:
    """Row tile of a step's expert segments for experts stored as ``fmt``.  Both halves of an exchange derive it from
    the same arguments: the planner pads every expert's segment to it and the grouped GEMMs walk the tiles with it.
    Quantised experts read their packed weights directly up to 64-row tiles; 128-row tiles mean the layer's experts are
    expanded to bf16 first, which only pays once every expert sees at least 64 rows on average."""
    t = pick_tile_rows(T, top_k, num_experts)
    if fmt != "bf16" and t == 128 and T * top_k < 64 * num_experts:
        t = 64
    return t


def wire_fp8_ok(geo: "ExchangeGeometry", tile_rows: int) -> bool:
    """Whether a step's rows travel as E4M3 + per-128 scales: the block-scaled expert GEMM consumes them as they are
    (decode-sized tiles); prefill-sized steps expand the experts to bf16 and want bf16 rows.  Both sides of the
    exchange call this with the same arguments."""
    return tile_rows < 128 and geo.hidden % 128 == 0


@dataclass
class ExchangeGeometry:
    hidden: int
    expert_ffn: int
    num_experts: int
    top_k: int
    max_tokens: int
    n_expert_ranks: int = 1
    # Waves: a step with more than ``wave_tokens`` tokens is exchanged as several independent sub-exchanges (own slab
    # region, plan block and flags each), so that the transfer of wave w+1 overlaps the expert GEMMs of wave w and the
    # return of wave w-1.  0 = one exchange per step.  The reference pipelines prefill the same way (units x waves,
    # rust/crates/cuteafd-daemon/src/shared/spark_waves.rs:1188-1517).
    wave_tokens: int = 0

    def rank_experts(self, r: int) -> tuple[int, int]:
        return expert_range(self.num_experts, self.n_expert_ranks, r)

    @property
    def regions(self) -> int:
        """Slab regions (= maximum number of waves of one step)."""
        return 1 if self.wave_tokens <= 0 else max(1, -(-self.max_tokens // self.wave_tokens))

    def region(self) -> "ExchangeGeometry":
        """Geometry of one region: what the plan / dispatch / grouped GEMM kernels of one wave see."""
        if self.wave_tokens <= 0 or self.wave_tokens >= self.max_tokens:
            return ExchangeGeometry(self.hidden, self.expert_ffn, self.num_experts, self.top_k, self.max_tokens, self.n_expert_ranks)
        return ExchangeGeometry(self.hidden, self.expert_ffn, self.num_experts, self.top_k, self.wave_tokens, self.n_expert_ranks)

    def waves(self, T: int) -> list[tuple[int, int]]:
        """Token ranges of the waves of a step with T tokens (every rank derives the same list)."""
        if self.wave_tokens <= 0 or T <= self.wave_tokens:
            return [(0, T)]
        n = -(-T // self.wave_tokens)
        per = -(-T // n)
        per = -(-per // 128) * 128                     # whole 128-row tiles per wave
        return [(a, min(T, a + per)) for a in range(0, T, per)]

    @property
    def max_rows(self) -> int:
        """Worst-case slab rows on one rank: every route lands there, plus tile padding."""
        per_rank = max(hi - lo for lo, hi in (self.rank_experts(r) for r in range(self.n_expert_ranks)))
        return self.max_tokens * self.top_k + per_rank * 128

    @property
    def max_tiles(self) -> int:
        return self.max_rows // 16 + 1

    @property
    def meta_ints(self) -> int:
        return 16 + 2 * self.max_tiles + self.max_rows


class ExpertSide:
    """Buffers an expert rank owns: the receive slab, the fc1 output and the plan meta block."""
    _dq_scratch: dict = {}           # per device: one layer's experts expanded to bf16 (shared by all regions)

    def __init__(self, geo: ExchangeGeometry, device: torch.device, slab: torch.Tensor | None = None,
                 meta: torch.Tensor | None = None, flags: torch.Tensor | None = None, num_layers: int = 1):
        self.geo = geo
        self.slab = slab if slab is not None else torch.zeros(geo.max_rows, geo.hidden, dtype=torch.bfloat16, device=device)
        self.meta = meta if meta is not None else torch.zeros(geo.meta_ints, dtype=torch.int32, device=device)
        self.flags = flags if flags is not None else torch.zeros(num_layers, dtype=torch.int32, device=device)
        self.hbuf = torch.zeros(geo.max_rows, geo.expert_ffn, dtype=torch.bfloat16, device=device)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        mt = geo.max_tiles
        self.num_tiles = self.meta[0:1]
        self.tile_expert = self.meta[16:16 + mt]
        self.tile_row0 = self.meta[16 + mt:16 + 2 * mt]
        self.row_dst = self.meta[16 + 2 * mt:]
        # E4M3 wire format: the same receive slab read as [max_rows, H] bytes followed by [max_rows, H / 128] fp32 scales
        # (fits: H + H / 32 bytes per row against 2 H for bf16), so a step may arrive in either form.
        if geo.hidden % 128 == 0:
            raw = self.slab.view(-1).view(torch.uint8)
            nq = geo.max_rows * geo.hidden
            self.wire_q = raw[:nq].view(torch.float8_e4m3fn).view(geo.max_rows, geo.hidden)
            self.wire_s = raw[nq:nq + geo.max_rows * (geo.hidden // 128) * 4].view(torch.float32).view(geo.max_rows, geo.hidden // 128)

    def run(self, w_gate: torch.Tensor, w_up: torch.Tensor, w_down: torch.Tensor, tile_rows: int, layer: int,
            epoch: torch.Tensor, combine_ptr: int, combine_flag_ptr: int | None, wait: bool) -> None:
        """fc1+SwiGLU then fc2 with the (token, slot) scatter into the attention rank's buffer."""
        g = self.geo
        K.grouped_linear(self.slab, w_gate, self.hbuf, self.tile_expert, self.tile_row0, self.num_tiles, g.max_tiles,
                         tile_rows, w_up=w_up, epoch=epoch,
                         wait_flag=(self.flags.data_ptr() + 4 * layer) if wait else None)
        K.grouped_linear(self.hbuf, w_down, self.hbuf, self.tile_expert, self.tile_row0, self.num_tiles, g.max_tiles,
                         tile_rows, row_dst=self.row_dst, out_ptr=combine_ptr, ldo=g.hidden, epoch=epoch,
                         signal_flag=combine_flag_ptr, done_counter=self.done[0:1] if combine_flag_ptr else None)


    def run_fp8(self, w_gate, w_up, w_down, tile_rows: int, rows: int, layer: int, epoch: torch.Tensor, combine_ptr: int,
                combine_flag_ptr: int | None, wait: bool, reuse_dequant: bool = False, wire: bool = False) -> None:
        """E4M3 experts: ``w_*`` = (values [E, N, K], scales [E, N/128, K/128]).  Received rows and the
        fc1 output are quantised 1x128 here, next to the GEMMs that consume them; with ``wire`` the rows arrived
        quantised by the dispatch (``wire_q`` / ``wire_s``) and fc1 itself waits for the dispatch flag."""
        g = self.geo
        if tile_rows == 128:
            # Prefill-sized step: the block-scaled kernel folds scales in its epilogue warps and falls behind the bf16
            # kernel at large row counts, so this layer's experts are expanded to bf16 (one layer's worth of scratch,
            # reused by every layer) and the bf16 grouped GEMMs run instead.
            dq = ExpertSide._dq_scratch.get(w_gate[0].device)
            if dq is None or dq[0].shape != w_gate[0].shape:
                dq = tuple(torch.empty(w[0].shape, dtype=torch.bfloat16, device=w[0].device) for w in (w_gate, w_up, w_down))
                ExpertSide._dq_scratch[w_gate[0].device] = dq
            self._dq = dq
            if not reuse_dequant:                # later waves of the same layer find the expanded weights in place
                for w, o in zip((w_gate, w_up, w_down), self._dq):
                    K.fp8_dequant_block128(w[0], w[1], o)
            self.run(self._dq[0], self._dq[1], self._dq[2], tile_rows, layer, epoch, combine_ptr, combine_flag_ptr, wait)
            return
        if not hasattr(self, "slab_q"):
            dev = self.slab.device
            self.slab_q = torch.zeros(g.max_rows, g.hidden, dtype=torch.float8_e4m3fn, device=dev)
            self.slab_s = torch.ones(g.max_rows, g.hidden // 128, dtype=torch.float32, device=dev)
            self.h_q = torch.zeros(g.max_rows, g.expert_ffn, dtype=torch.float8_e4m3fn, device=dev)
            self.h_s = torch.ones(g.max_rows, g.expert_ffn // 128, dtype=torch.float32, device=dev)
        rows = min(rows, g.max_rows)
        if wire:
            K.grouped_linear_fp8(self.wire_q, self.wire_s, w_gate[0], w_gate[1], self.hbuf, self.tile_expert, self.tile_row0,
                                 self.num_tiles, g.max_tiles, tile_rows, w_up=w_up[0], ws_up=w_up[1], epoch=epoch,
                                 wait_flag=(self.flags.data_ptr() + 4 * layer) if wait else None)
        else:
            if wait:
                K.wait_flag(self.flags.data_ptr() + 4 * layer, epoch)
            K.quant_rows_fp8(self.slab[:rows], self.slab_q[:rows], self.slab_s[:rows])
            K.grouped_linear_fp8(self.slab_q, self.slab_s, w_gate[0], w_gate[1], self.hbuf, self.tile_expert, self.tile_row0,
                                 self.num_tiles, g.max_tiles, tile_rows, w_up=w_up[0], ws_up=w_up[1])
        K.quant_rows_fp8(self.hbuf[:rows], self.h_q[:rows], self.h_s[:rows])
        K.grouped_linear_fp8(self.h_q, self.h_s, w_down[0], w_down[1], self.hbuf, self.tile_expert, self.tile_row0,
                             self.num_tiles, g.max_tiles, tile_rows, row_dst=self.row_dst, out_ptr=combine_ptr, ldo=g.hidden,
                             epoch=epoch, signal_flag=combine_flag_ptr,
                             done_counter=self.done[0:1] if combine_flag_ptr else None)

    def run_w4(self, fmt: str, w_gate, w_up, w_down, tile_rows: int, layer: int, epoch: torch.Tensor, combine_ptr: int,
               combine_flag_ptr: int | None, wait: bool) -> None:
        """MXFP4 / NVFP4 experts (decode-sized tiles, <= 64 rows): ``w_*`` = (packed [E, N, K/2], block scales, global
        scales [E] or None).  Weights are expanded inside the grouped GEMMs; activations stay bf16."""
        g = self.geo
        assert tile_rows <= 64
        K.grouped_linear_w4(self.slab, w_gate, fmt, self.hbuf, self.tile_expert, self.tile_row0, self.num_tiles, g.max_tiles,
                            tile_rows, w_up=w_up, wait_flag=(self.flags.data_ptr() + 4 * layer) if wait else None,
                            epoch=epoch if wait else None)
        K.grouped_linear_w4(self.hbuf, w_down, fmt, self.hbuf, self.tile_expert, self.tile_row0, self.num_tiles, g.max_tiles,
                            tile_rows, row_dst=self.row_dst, out_ptr=combine_ptr, ldo=g.hidden, epoch=epoch,
                            signal_flag=combine_flag_ptr, done_counter=self.done[0:1] if combine_flag_ptr else None)


    def run_w4_any(self, fmt: str, w_gate, w_up, w_down, tile_rows: int, layer: int, epoch: torch.Tensor, combine_ptr: int,
                   combine_flag_ptr: int | None, reuse_dequant: bool = False, wait: bool = True) -> None:
        """MXFP4 / NVFP4 experts at any step size: decode-sized tiles read the packed weights directly; prefill-sized
        steps expand this layer's experts to bf16 once (one layer's worth of scratch, shared by all layers) and take
        the bf16 grouped GEMMs."""
        if tile_rows <= 64:
            return self.run_w4(fmt, w_gate, w_up, w_down, tile_rows, layer, epoch, combine_ptr, combine_flag_ptr, wait=wait)
        dev = w_gate[0].device
        shapes = [(*w[0].shape[:-1], w[0].shape[-1] * 2) for w in (w_gate, w_up, w_down)]
        dq = ExpertSide._dq_scratch.get(dev)
        if dq is None or [tuple(t.shape) for t in dq] != [tuple(sh) for sh in shapes]:
            dq = tuple(torch.empty(sh, dtype=torch.bfloat16, device=dev) for sh in shapes)
            ExpertSide._dq_scratch[dev] = dq
        if not reuse_dequant:
            for w, o in zip((w_gate, w_up, w_down), dq):
                K.w4_dequant(w, fmt, out=o)
        self.run(dq[0], dq[1], dq[2], tile_rows, layer, epoch, combine_ptr, combine_flag_ptr, wait)


class AttentionSide:
    """Buffers the attention rank owns: routes, plan output, the combine buffer and its flags."""

    def __init__(self, geo: ExchangeGeometry, device: torch.device, combine: torch.Tensor | None = None,
                 flags: torch.Tensor | None = None, num_layers: int = 1):
        self.geo = geo
        T, k = geo.max_tokens, geo.top_k
        self.idx = torch.zeros(T, k, dtype=torch.int32, device=device)
        self.w = torch.zeros(T, k, dtype=torch.float32, device=device)
        self.dest_row = torch.zeros(T * k, dtype=torch.int32, device=device)
        self.combine = combine if combine is not None else torch.zeros(T * k, geo.hidden, dtype=torch.bfloat16, device=device)
        # one word per (layer, expert rank), written by that rank's fc2 kernel
        self.flags = flags if flags is not None else torch.zeros(num_layers * _n.MAX_RANKS, dtype=torch.int32, device=device)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)
        self.expert_count = torch.zeros(geo.num_experts, dtype=torch.int32, device=device)
        self.layout = _n.MoeLayout()
        self.layout.n_ranks = geo.n_expert_ranks
        for r in range(geo.n_expert_ranks):
            self.layout.expert_lo[r] = geo.rank_experts(r)[0]
        for r in range(geo.n_expert_ranks, _n.MAX_RANKS + 1):
            self.layout.expert_lo[r] = geo.num_experts
        self.layout.max_tiles, self.layout.max_rows = geo.max_tiles, geo.max_rows
        self._rank_ptrs: list[tuple[int, int, int]] = []

    def bind_rank(self, r: int, slab_ptr: int, meta_ptr: int, flags_ptr: int) -> None:
        """Record rank r's slab / meta / per-layer dispatch flag base (local or peer addresses)."""
        while len(self._rank_ptrs) <= r:
            self._rank_ptrs.append((0, 0, 0))
        self._rank_ptrs[r] = (slab_ptr, meta_ptr, flags_ptr)
        self.layout.slab[r], self.layout.meta[r] = slab_ptr, meta_ptr
        # the E4M3 wire form of the same slab: bytes first, then the per-128 scales (``ExpertSide.wire_q`` / ``wire_s``)
        self.layout.slab_q[r] = slab_ptr
        self.layout.slab_s[r] = slab_ptr + self.geo.max_rows * self.geo.hidden

    # Plan and dispatch share one single-block launch only while one SM can copy the rows faster than a second launch
    # costs: measured in a CUDA graph, Qwen3 rows (4 KB) 8.5 vs 13.0 us at 1 token but 28.7 vs 18.3 us at 32; DeepSeek-V3
    # rows (14 KB) 11.5 vs 13.2 us at 1 token, 25.7 vs 14.9 us at 8, 143 vs 20 us at 64.  Rows quantised on the wire
    # always take the separate dispatch kernel (the single block would quantise them all: 18.5 vs 14.5 us at 1 token).
    FUSED_DISPATCH_ROWS = 512
    FUSED_DISPATCH_BYTES = 128 << 10

    def dispatch(self, x: torch.Tensor, logits: torch.Tensor | None, route_kw: dict, tile_rows: int, layer: int,
                 epoch: torch.Tensor, wire_fp8: bool = False) -> None:
        """Route (unless ``logits`` is None: then ``idx`` / ``w`` were already filled by ``norm_route``), plan, and
        copy the rows into the owners' slabs; ``wire_fp8`` sends them as E4M3 + per-128 scales."""
        T = x.shape[0]
        g = self.geo
        self.layout.fp8 = int(wire_fp8)
        idx, w = self.idx[:T], self.w[:T]
        if logits is not None:
            K.route_topk(logits, g.top_k, out_idx=idx, out_w=w, **route_kw)
        for r in range(g.n_expert_ranks):
            self.layout.flag[r] = self._rank_ptrs[r][2] + 4 * layer
        if (T * g.top_k <= self.FUSED_DISPATCH_ROWS and T * g.top_k * g.hidden * 2 <= self.FUSED_DISPATCH_BYTES
                and not wire_fp8):
            K.moe_plan(idx, g.num_experts, tile_rows, self.layout, self.dest_row, self.expert_count, x=x, epoch=epoch)
        else:
            K.moe_plan(idx, g.num_experts, tile_rows, self.layout, self.dest_row, self.expert_count)
            K.moe_dispatch(x, idx, self.dest_row, self.layout, epoch, self.done[0:1])

    def combine_into(self, out: torch.Tensor, T: int, layer: int, epoch: torch.Tensor, *,
                     shared: torch.Tensor | None, residual: torch.Tensor | None, wait: bool,
                     norm_w: torch.Tensor | None = None, eps: float = 0.0, x_out: torch.Tensor | None = None) -> torch.Tensor:
        g = self.geo
        flags_ptr = self.flags.data_ptr() + 4 * layer * _n.MAX_RANKS if wait else None
        return K.moe_combine(self.combine, self.w[:T], out, shared=shared, residual=residual, flags_ptr=flags_ptr,
                             n_flags=g.n_expert_ranks if wait else 0, epoch=epoch, norm_w=norm_w, eps=eps, x_out=x_out)


class LocalExchange:
    """Single-GPU MoE: attention side and expert side in one process, stream-ordered."""

    def __init__(self, geo: ExchangeGeometry, device: torch.device):
        assert geo.n_expert_ranks == 1
        self.geo = geo
        self.att = AttentionSide(geo, device)
        self.exp = ExpertSide(geo, device)
        self.att.bind_rank(0, self.exp.slab.data_ptr(), self.exp.meta.data_ptr(), self.exp.flags.data_ptr())
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)

    def forward(self, x: torch.Tensor, logits: torch.Tensor, route_kw: dict, w_gate: torch.Tensor, w_up: torch.Tensor,
                w_down: torch.Tensor, out: torch.Tensor, *, shared: torch.Tensor | None = None,
                residual: torch.Tensor | None = None, tile_rows: int | None = None, norm_w: torch.Tensor | None = None,
                eps: float = 0.0, x_out: torch.Tensor | None = None) -> torch.Tensor:
        """``logits`` None = the routes are already in ``self.att.idx`` / ``self.att.w`` (``norm_route``).  ``norm_w`` /
        ``x_out`` fuse the next layer's input RMSNorm into the combine."""
        T = x.shape[0]
        g = self.geo
        tile_rows = tile_rows or pick_tile_rows(T, g.top_k, g.num_experts)
        self.att.dispatch(x, logits, route_kw, tile_rows, 0, self.epoch)
        self.exp.run(w_gate, w_up, w_down, tile_rows, 0, self.epoch, self.att.combine.data_ptr(), None, wait=False)
        return self.att.combine_into(out, T, 0, self.epoch, shared=shared, residual=residual, wait=False, norm_w=norm_w,
                                     eps=eps, x_out=x_out)

    def forward_fp8(self, x: torch.Tensor, logits: torch.Tensor, route_kw: dict, w_gate, w_up, w_down, out: torch.Tensor, *,
                    shared: torch.Tensor | None = None, residual: torch.Tensor | None = None,
                    tile_rows: int | None = None, wire: bool | None = None) -> torch.Tensor:
        """Same exchange with E4M3 experts: each ``w_*`` is (values [E, N, K] e4m3, scales [E, N/128, K/128]).
        Decode-sized steps quantise the rows 1x128 inside the dispatch (``wire``); otherwise on the expert side before
        each grouped GEMM."""
        T = x.shape[0]
        g = self.geo
        tile_rows = tile_rows or plan_tile_rows("fp8", T, g.top_k, g.num_experts)
        wire = wire_fp8_ok(g, tile_rows) if wire is None else wire
        self.att.dispatch(x, logits, route_kw, tile_rows, 0, self.epoch, wire_fp8=wire)
        e = self.exp
        if tile_rows == 128:
            # prefill-sized step: expand this layer's experts to bf16 once and take the bf16 grouped GEMMs
            e.run_fp8(w_gate, w_up, w_down, tile_rows, 0, 0, self.epoch, self.att.combine.data_ptr(), None, wait=False)
            return self.att.combine_into(out, T, 0, self.epoch, shared=shared, residual=residual, wait=False)
        rows = min(g.max_rows, T * g.top_k + g.num_experts * tile_rows)
        if not hasattr(e, "slab_q"):
            dev = e.slab.device
            e.slab_q = torch.zeros(g.max_rows, g.hidden, dtype=torch.float8_e4m3fn, device=dev)
            e.slab_s = torch.ones(g.max_rows, g.hidden // 128, dtype=torch.float32, device=dev)
            e.h_q = torch.zeros(g.max_rows, g.expert_ffn, dtype=torch.float8_e4m3fn, device=dev)
            e.h_s = torch.ones(g.max_rows, g.expert_ffn // 128, dtype=torch.float32, device=dev)
        if wire:
            xq, xs = e.wire_q, e.wire_s
        else:
            xq, xs = e.slab_q, e.slab_s
            K.quant_rows_fp8(e.slab[:rows], xq[:rows], xs[:rows])
        K.grouped_linear_fp8(xq, xs, w_gate[0], w_gate[1], e.hbuf, e.tile_expert, e.tile_row0, e.num_tiles,
                             g.max_tiles, tile_rows, w_up=w_up[0], ws_up=w_up[1])
        K.quant_rows_fp8(e.hbuf[:rows], e.h_q[:rows], e.h_s[:rows])
        K.grouped_linear_fp8(e.h_q, e.h_s, w_down[0], w_down[1], e.hbuf, e.tile_expert, e.tile_row0, e.num_tiles,
                             g.max_tiles, tile_rows, row_dst=e.row_dst, out_ptr=self.att.combine.data_ptr(), ldo=g.hidden)
        return self.att.combine_into(out, T, 0, self.epoch, shared=shared, residual=residual, wait=False)


def _forward_w4(self, fmt: str, x: torch.Tensor, logits: torch.Tensor, route_kw: dict, w_gate, w_up, w_down, out: torch.Tensor, *,
                shared: torch.Tensor | None = None, residual: torch.Tensor | None = None) -> torch.Tensor:
    """Local exchange with MXFP4 / NVFP4 experts.  Decode-sized steps run the weight-expanding grouped GEMM; larger
    ones expand the layer's experts to bf16 once and take the bf16 path."""
    T = x.shape[0]
    g = self.geo
    tile_rows = plan_tile_rows(fmt, T, g.top_k, g.num_experts)
    self.att.dispatch(x, logits, route_kw, tile_rows, 0, self.epoch)
    self.exp.run_w4_any(fmt, w_gate, w_up, w_down, tile_rows, 0, self.epoch, self.att.combine.data_ptr(), None, wait=False)
    return self.att.combine_into(out, T, 0, self.epoch, shared=shared, residual=residual, wait=False)


LocalExchange.forward_w4 = _forward_w4


def _forward_stored(self, fmt: str, x, logits, route_kw, w_gate, w_up, w_down, out, *, shared=None, residual=None, norm_w=None,
                    eps: float = 0.0, x_out=None):
    """One entry for every expert storage format ("bf16", "fp8", "mxfp4", "nvfp4"); the quantised forms do not fuse the
    next layer's norm into the combine, so the caller norms separately (returns whether ``x_out`` was written)."""
    if fmt == "bf16":
        self.forward(x, logits, route_kw, w_gate, w_up, w_down, out, shared=shared, residual=residual, norm_w=norm_w, eps=eps,
                     x_out=x_out)
        return norm_w is not None
    if fmt == "fp8":
        self.forward_fp8(x, logits, route_kw, w_gate, w_up, w_down, out, shared=shared, residual=residual)
    else:
        self.forward_w4(fmt, x, logits, route_kw, w_gate, w_up, w_down, out, shared=shared, residual=residual)
    return False


LocalExchange.forward_stored = _forward_stored
