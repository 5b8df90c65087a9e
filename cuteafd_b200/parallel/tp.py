"""Tensor parallelism for the attention ranks with the collectives fused into the kernels.

Residual rows are sharded over the TP ranks (rank r owns rows [r*R, (r+1)*R)); activations that a
column-parallel GEMM needs in full are all-gathered by *push*.

    y_partial = a_local @ W_row_shard.T          row-parallel GEMM whose epilogue stores every output
                                                 row into its owner's receive buffer (peer memory) and
                                                 raises the owner's flag        [GEMM -> reduce-scatter]
    h_own += sum_r partial_r ; x_own = norm(h)   owner waits for all flags, adds in rank order in fp32,
                                                 stores x_own into every rank's activation buffer and
                                                 raises their flags             [reduce + norm + all-gather]
    z_local = x_full @ W_col_shard.T             column-parallel GEMM that waits for those flags inside
                                                 the kernel and TMA-loads from local memory [all-gather -> GEMM]

No NCCL call sits on this path; NCCL is only the measured baseline (``baseline_*``).  The reference
does the degree-2 version with push / wait / ordered add kernels
(rust/crates/cuteafd-daemon/src/shared/peer_split.rs:1-14, native/shared/cuda/peer_exchange.cu:69-263).
"""
from __future__ import annotations

import ctypes as C

import torch
import torch.distributed as dist

from .._native import lib as _n
from ..ops import kernels as K
from .afd import GUARD, SymmetricHeap, _align


class TpContext:
    """Symmetric buffers + flags of one TP group for activations of width ``hidden``."""

    def __init__(self, hidden: int, max_rows: int, device: torch.device, group=None):
        self.group = group or dist.group.WORLD
        self.ranks, self.rank = dist.get_world_size(self.group), dist.get_rank(self.group)
        self.hidden, self.device = hidden, device
        self.rows_per_rank = self.max_rows_per_rank = (max_rows + self.ranks - 1) // self.ranks
        R, n = self.rows_per_rank, self.ranks
        o = 0
        bands = []

        def region(name: str, nbytes: int) -> int:                       # every region ends in a guard band
            nonlocal o
            start = o
            o = _align(o + nbytes) + GUARD
            bands.append((name, o - GUARD))
            return start
        self.off_partials = region("partials", n * R * hidden * 2)       # receive buffer [ranks][R][hidden]
        self.off_x = region("gathered activations", n * R * hidden * 2)  # [ranks*R][hidden]
        self.off_rs_flags = region("reduce-scatter flags", 64)
        self.off_ag_flags = region("all-gather flags", 64)
        self.off_ready_flags = region("ready flags", 64)
        self.off_head_flags = region("head flags", 64)
        self.head_rows = max(64, min(max_rows, 4096))                    # rows one sharded-head selection can cover
        self.off_head_table = region("head table", n * self.head_rows * 8)   # (value, id) per rank and row
        self.heap = SymmetricHeap(o, device, self.group)
        self.heap.arm(bands)
        torch.cuda.synchronize()
        dist.barrier(self.group)
        self.partials = self.heap.view(self.off_partials, n * R * hidden * 2, torch.bfloat16).view(n, R, hidden)
        self.x_full = self.heap.view(self.off_x, n * R * hidden * 2, torch.bfloat16).view(n * R, hidden)
        self.rs_flags = self.heap.view(self.off_rs_flags, 64, torch.int32)
        self.ag_flags = self.heap.view(self.off_ag_flags, 64, torch.int32)
        self.ready_flags = self.heap.view(self.off_ready_flags, 64, torch.int32)
        self.head_flags = self.heap.view(self.off_head_flags, 64, torch.int32)
        self.head_table = self.heap.view(self.off_head_table, n * self.head_rows * 8, torch.int64)
        self._head_cand = None
        self.head_epoch = torch.zeros(1, dtype=torch.int32, device=device)   # its own counter: ``epoch`` belongs to the step protocol
        self._ready_ptrs = (C.c_void_p * 8)(*[self.heap.ptrs[r] + self.off_ready_flags + 4 * self.rank for r in range(n)])
        self.residual = torch.zeros(R, hidden, dtype=torch.bfloat16, device=device)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=device)
        self.done = torch.zeros(4, dtype=torch.int32, device=device)

    def step(self) -> None:
        """One new epoch per collective round (all ranks call it the same number of times)."""
        K.bump_epoch(self.epoch)

    def rows_owned(self, total_rows: int) -> int:
        lo = self.rank * self.rows_per_rank
        return max(0, min(self.rows_per_rank, total_rows - lo))

    # ---- GEMM -> reduce-scatter -----------------------------------------------------------------------
    def row_parallel_linear(self, a_local: torch.Tensor, w_shard: torch.Tensor) -> None:
        """partial = a_local @ w_shard.T, each output row stored at its owner (flag raised at the end)."""
        T, Kd = a_local.shape
        N = w_shard.shape[0]
        assert N == self.hidden and T <= self.ranks * self.rows_per_rank
        a = _n.GemmArgs()
        a.w0, a.x, a.out = w_shard.data_ptr(), a_local.data_ptr(), self.partials.data_ptr()
        a.status = K.status_word(self.device).data_ptr()
        a.w_rows_total, a.x_rows_total = N, T
        a.k, a.n_features, a.x_rows, a.ldo = Kd, N, T, N
        swap = T <= 128
        a.swap, a.dual, a.bx = int(swap), 0, (K.pick_token_tile(T) if swap else 128)
        a.num_sms = K.num_sms()
        a.rs_ranks, a.rs_rows_per_rank, a.rs_my_rank = self.ranks, self.rows_per_rank, self.rank
        for r in range(self.ranks):
            a.rs_out[r] = self.heap.ptrs[r] + self.off_partials
            a.signal_flags[r] = self.heap.ptrs[r] + self.off_rs_flags + 4 * self.rank
        a.n_signal_flags = self.ranks
        a.epoch, a.done_counter = self.epoch.data_ptr(), self.done[0:1].data_ptr()
        _n.check(_n.cuda_lib().cafd_gemm(C.byref(a), K._stream()), "cafd_gemm(reduce-scatter)")

    # ---- reduce + residual + norm + all-gather -----------------------------------------------------------
    def reduce_norm_gather(self, total_rows: int, norm_w: torch.Tensor, eps: float, local: torch.Tensor | None = None,
                           gather_only: bool = False) -> None:
        """Owned rows: residual += sum of every rank's partial (rank order, fp32, one rounding), x = norm(residual),
        x stored into every rank's ``x_full`` and the gather flags raised.  ``local`` [rows owned, hidden] replaces
        the partials by a rank-local addend (the FFN output of the owned rows: nothing to wait for);
        ``gather_only`` adds nothing (first norm of a step)."""
        a = _n.TpReduceArgs()
        a.residual, a.norm_w = self.residual.data_ptr(), norm_w.data_ptr()
        if gather_only:
            a.partials, a.n_sum, a.n_wait = self.partials.data_ptr(), 0, 0
        elif local is not None:
            assert local.is_contiguous() and local.shape[1] == self.hidden and local.shape[0] >= self.rows_owned(total_rows)
            a.partials, a.n_sum, a.n_wait = local.data_ptr(), 1, 0
        else:
            a.partials, a.n_sum, a.n_wait = self.partials.data_ptr(), self.ranks, self.ranks
        for r in range(self.ranks):
            a.x_out[r] = self.heap.ptrs[r] + self.off_x
            a.ag_flags[r] = self.heap.ptrs[r] + self.off_ag_flags + 4 * self.rank
        a.rs_flags, a.epoch, a.done_counter = self.rs_flags.data_ptr(), self.epoch.data_ptr(), self.done[1:2].data_ptr()
        a.status = K.status_word(self.device).data_ptr()
        a.ranks, a.my_rank, a.rows_per_rank, a.rows_valid, a.N, a.eps = (self.ranks, self.rank, self.rows_per_rank,
                                                                      self.rows_owned(total_rows), self.hidden, eps)
        _n.check(_n.cuda_lib().cafd_tp_reduce_norm_gather(C.byref(a), K._stream()), "tp_reduce_norm_gather")

    def set_rows(self, total_rows: int) -> None:
        """Row ownership of the coming step: rank r owns rows [r * R, (r + 1) * R) with R = ceil(total_rows / ranks), so
        small steps are shared evenly too.  Every rank must call it with the same value."""
        r = (total_rows + self.ranks - 1) // self.ranks
        assert 0 < r <= self.max_rows_per_rank
        self.rows_per_rank = r

    def release_buffers(self) -> None:
        """End of a step: this rank's reads of the gathered activations are done (stream order); tell every rank."""
        _n.check(_n.cuda_lib().cafd_tp_signal(self._ready_ptrs, self.ranks, self.epoch.data_ptr(), K._stream()), "tp_signal")

    def wait_buffers_free(self) -> None:
        """Start of a step, before the epoch moves: wait until every rank has released the previous step's buffers."""
        for r in range(self.ranks):
            K.wait_flag(self.ready_flags.data_ptr() + 4 * r, self.epoch)

    def wait_gathered(self) -> None:
        """Stream-ordered wait until every rank's rows of ``x_full`` have arrived (for readers that are not the
        flag-waiting GEMM)."""
        for r in range(self.ranks):
            K.wait_flag(self.ag_flags.data_ptr() + 4 * r, self.epoch)

    # ---- vocabulary-sharded head: candidates only cross the fabric ------------------------------------------------
    def head_pick(self, local_logits: torch.Tensor, lo: int, out: torch.Tensor) -> torch.Tensor:
        """Greedy ids [T] from this rank's slice of the logits ([T, hi - lo] fp32, global ids lo..hi): per-slice
        candidates, then one kernel that exchanges (value, id) with every rank and picks (ties to the lowest id).
        Every rank calls it for the same rows, the same number of times (the exchange counts its own rounds)."""
        T, V = local_logits.shape
        assert 0 < T <= self.head_rows and local_logits.dtype == torch.float32
        L = _n.cuda_lib()
        slices = L.cafd_argmax_slices()
        if self._head_cand is None:
            self._head_cand = (torch.empty(self.head_rows * slices, dtype=torch.float32, device=self.device),
                               torch.empty(self.head_rows * slices, dtype=torch.int32, device=self.device))
        cv, ci = self._head_cand
        if V > 0:
            _n.check(L.cafd_argmax_candidates(local_logits.data_ptr(), cv.data_ptr(), ci.data_ptr(), T, V, local_logits.stride(0),
                                              K._stream()), "argmax_candidates")
        else:                                                            # a rank past the end of the vocabulary never wins
            cv[:T * slices].fill_(float("-inf")); ci[:T * slices].fill_(0x7fffffff)
        K.bump_epoch(self.head_epoch)
        a = _n.TpHeadArgs()
        a.cand_v, a.cand_i = cv.data_ptr(), ci.data_ptr()
        for r in range(self.ranks):
            a.table_out[r] = self.heap.ptrs[r] + self.off_head_table
            a.flags_out[r] = self.heap.ptrs[r] + self.off_head_flags + 4 * self.rank
        a.table_in, a.flags_in = self.head_table.data_ptr(), self.head_flags.data_ptr()
        a.epoch, a.done_counter, a.status = self.head_epoch.data_ptr(), self.done[2:3].data_ptr(), K.status_word(self.device).data_ptr()
        a.out = out.data_ptr()
        a.ranks, a.my_rank, a.max_rows, a.T, a.slices, a.lo = self.ranks, self.rank, self.head_rows, T, slices, lo
        _n.check(L.cafd_tp_head_pick(C.byref(a), K._stream()), "tp_head_pick")
        return out

    # ---- all-gather -> GEMM -----------------------------------------------------------------------------------
    def column_parallel_linear(self, total_rows: int, w_shard: torch.Tensor, out: torch.Tensor, w_up: torch.Tensor | None = None) -> torch.Tensor:
        """out = x_full[:total_rows] @ w_shard.T, waiting inside the kernel for every rank's gathered rows."""
        Kd, N = self.hidden, w_shard.shape[0]
        a = _n.GemmArgs()
        a.w0, a.w1, a.x, a.out = w_shard.data_ptr(), (w_up.data_ptr() if w_up is not None else None), self.x_full.data_ptr(), out.data_ptr()
        a.status = K.status_word(self.device).data_ptr()
        a.w_rows_total, a.x_rows_total = N, total_rows
        a.k, a.n_features, a.x_rows, a.ldo = Kd, N, total_rows, out.stride(0)
        swap = total_rows <= 128
        a.swap, a.dual, a.bx = int(swap), int(w_up is not None), (K.pick_token_tile(total_rows) if swap else 128)
        a.num_sms = K.num_sms()
        a.wait_flag, a.n_wait_flags, a.epoch = self.ag_flags.data_ptr(), self.ranks, self.epoch.data_ptr()
        _n.check(_n.cuda_lib().cafd_gemm(C.byref(a), K._stream()), "cafd_gemm(all-gather)")
        return out

    # ---- NCCL baseline twins -------------------------------------------------------------------------------------
    def baseline_block(self, a_local: torch.Tensor, w_row: torch.Tensor, residual_own: torch.Tensor, norm_w: torch.Tensor,
                       eps: float, w_col: torch.Tensor) -> tuple[torch.Tensor, torch.Tensor]:
        """cuBLAS + NCCL reduce-scatter + all-gather version of the same three steps."""
        from ..ref import ops as R
        T = a_local.shape[0]
        partial = a_local @ w_row.T
        pad = self.ranks * self.rows_per_rank - T
        if pad:
            partial = torch.cat([partial, partial.new_zeros(pad, partial.shape[1])])
        own = torch.empty(self.rows_per_rank, self.hidden, dtype=partial.dtype, device=partial.device)
        dist.reduce_scatter_tensor(own, partial, group=self.group)
        h = (residual_own.float() + own.float()).to(torch.bfloat16)
        x = R.rmsnorm(h, norm_w, eps)
        full = torch.empty(self.ranks * self.rows_per_rank, self.hidden, dtype=x.dtype, device=x.device)
        dist.all_gather_into_tensor(full, x, group=self.group)
        return h, full[:T] @ w_col.T
