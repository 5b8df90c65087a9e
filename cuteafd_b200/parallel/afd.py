"""Attention/FFN disaggregation over one NVLink domain: ranks 0..A-1 run the backbone (attention,
router, head, KV cache) as data-parallel replicas, each serving its own sequences; ranks A..N-1
hold the routed experts, partitioned by expert id, and serve every replica.  A = 1 is the plain
"one attention rank + expert ranks" deployment; A = 2 with six expert ranks is the reference's
"two coordinator GPUs + six expert boxes" shape (rust/crates/cuteafd-loader/src/placement/mod.rs:303-311
splits heads between its two coordinators because a 96 GB card cannot hold the backbone twice; with
180 GB per GPU each replica holds the whole backbone and no per-layer collective joins them).

Data path (no NCCL, no host hop): every rank maps one symmetric buffer of every other rank
(``torch.distributed._symmetric_memory`` does the handle exchange).  The attention rank's plan and
dispatch kernels store tile lists and token rows straight into the owners' buffers and publish a
per-layer step number; the owners' grouped tcgen05 GEMMs wait for it, and the fc2 epilogue stores
each (token, slot) row straight into the attention rank's combine buffer and publishes the step
number back; the combine kernel waits for every owner.  Kernel waits are bounded and report
through the status word.

Control path: one small NCCL broadcast per forward call (op, steps, tokens of every replica) so
expert ranks know how many layer sequences to launch and for which sources; a run of decode steps
is announced once and then proceeds on device flags only.  Replicas run the same script in step:
replica 0 sends every announcement (it knows, from the script, how many tokens each replica brings),
the other replicas receive it where replica 0 sends it, and a replica with nothing to do in a round
waits in ``end_round`` until replica 0 closes the round.

The reference's coordinator/expertd split over RoCE is the same idea with a host transport worker
in the middle (rust/crates/cuteafd-daemon/src/shared/experts/service.rs:22-135;
rust/crates/cuteafd-daemon/src/shared/spark_waves.rs:1188-1517).
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from .._native import lib as _n
from ..config import ModelConfig
from ..ops import kernels as K
from .moe_exchange import AttentionSide, ExchangeGeometry, ExpertSide, pick_tile_rows, plan_tile_rows, wire_fp8_ok

OP_STOP, OP_STEPS, OP_TIMED, OP_SYNC = 0, 1, 2, 3


def _align(x: int, a: int = 1024) -> int:
    return (x + a - 1) // a * a


# Guard band after every region of a symmetric buffer that peers write into: filled with a pattern when the buffer is
# created, looked at by ``SymmetricHeap.damaged()`` (tests, round ends, shutdown).  A kernel that stores past its region
# (a row index beyond the slab, a flag slot beyond the table) lands in a band instead of in its neighbour's data, and
# the damage names the region.  The reference guards its exchange buffers with sanitizer builds and poisoned padding
# (native/CMakeLists.txt sanitizer options; native/shared/src/cuteafd_native.cc buffer registration).
GUARD = 1024
GUARD_BYTE = 0xA5


@dataclass
class SymLayout:
    """Byte offsets inside every rank's symmetric buffer (same layout on all ranks)."""
    slab: int
    meta: int
    dflags: int      # per-layer dispatch flags (written by the attention rank)
    combine: int
    cflags: int      # per-(layer, rank) completion flags (written by expert ranks)
    total: int

    @staticmethod
    def build(geo: ExchangeGeometry, num_layers: int, n_sources: int = 1) -> "SymLayout":
        """Per source (attention replica) ``geo.regions`` slab regions and plan blocks (one per wave of a large step)
        and one dispatch flag per (layer, source, wave): region = source * regions + wave, flag slot = layer *
        (sources * regions) + region.  The combine buffer and its completion flags [layer, wave, expert rank] belong
        to the rank that owns them, so they need no source dimension."""
        rg, n = geo.region(), geo.regions * n_sources
        o = 0
        slab = o; o = _align(o + n * SymLayout.slab_stride(geo))
        meta = o; o = _align(o + n * SymLayout.meta_stride(geo))
        dflags = o; o = _align(o + num_layers * n * 4) + GUARD
        combine = o; o = _align(o + geo.max_tokens * geo.top_k * geo.hidden * 2) + GUARD
        cflags = o; o = _align(o + num_layers * geo.regions * _n.MAX_RANKS * 4) + GUARD
        return SymLayout(slab, meta, dflags, combine, cflags, o)

    @staticmethod
    def slab_stride(geo: ExchangeGeometry) -> int:
        return _align(geo.region().max_rows * geo.hidden * 2) + GUARD

    @staticmethod
    def meta_stride(geo: ExchangeGeometry) -> int:
        return _align(geo.region().meta_ints * 4) + GUARD

    def guards(self, geo: ExchangeGeometry, n_sources: int = 1) -> list[tuple[str, int]]:
        """(name, byte offset) of every guard band: the last ``GUARD`` bytes of each slab region and plan block, and of
        the dispatch-flag table, the combine buffer and the completion-flag table."""
        n = geo.regions * n_sources
        out = [(f"slab[{r}]", self.slab + (r + 1) * self.slab_stride(geo) - GUARD) for r in range(n)]
        out += [(f"meta[{r}]", self.meta + (r + 1) * self.meta_stride(geo) - GUARD) for r in range(n)]
        out += [("dispatch flags", self.combine - GUARD), ("combine", self.cflags - GUARD), ("completion flags", self.total - GUARD)]
        return out


class SymmetricHeap:
    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        try:
            self.handle = symm_mem.rendezvous(self.buf, group)
        except Exception:
            # older runtimes want the group registered first
            symm_mem.enable_symm_mem_for_group(group.group_name)
            self.handle = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        self.bands: list[tuple[str, int]] = []
        torch.cuda.synchronize()
        dist.barrier()

    def view(self, offset: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        return self.buf[offset:offset + nbytes].view(dtype)

    def arm(self, bands: list[tuple[str, int]]) -> None:
        """Fill the guard bands (before any peer writes: the constructor's barrier has passed, no step has run)."""
        self.bands = list(bands)
        for _, off in self.bands:
            self.buf[off:off + GUARD].fill_(GUARD_BYTE)

    def damaged(self) -> list[str]:
        """Names of the guard bands a store has landed in (one small device read per band; not on the step path)."""
        if not self.bands:
            return []
        idx = torch.tensor([off for _, off in self.bands], device=self.buf.device)
        rows = self.buf[(idx[:, None] + torch.arange(GUARD, device=self.buf.device)[None, :]).view(-1)].view(len(self.bands), GUARD)
        bad = (rows != GUARD_BYTE).any(dim=1).tolist()
        return [name for (name, _), b in zip(self.bands, bad) if b]


class RemoteExchange:
    """Attention-rank half: same interface as ``LocalExchange`` with experts on other GPUs.  A step larger than
    ``geo.wave_tokens`` goes out as several waves (own slab region / plan block / flags each)."""

    def __init__(self, geo: ExchangeGeometry, heap: SymmetricHeap, lay: SymLayout, num_layers: int, source: int = 0,
                 n_sources: int = 1):
        """``source``: this replica's index among the ``n_sources`` attention ranks (= its global rank); expert rank r
        is global rank n_sources + r."""
        dev = heap.buf.device
        self.geo, self.heap, self.lay = geo, heap, lay
        self.source, self.n_sources = source, n_sources
        self.expert_format = "bf16"              # how the expert ranks hold their weights: decides the row tile of a plan
        rg, n = geo.region(), geo.regions
        self.combine = heap.view(lay.combine, geo.max_tokens * geo.top_k * geo.hidden * 2, torch.bfloat16).view(-1, geo.hidden)
        cflags = heap.view(lay.cflags, num_layers * n * _n.MAX_RANKS * 4, torch.int32)
        self.sides: list[AttentionSide] = []
        for w in range(n):
            side = AttentionSide(rg, dev, combine=self.combine, flags=cflags, num_layers=num_layers * n)
            region = source * n + w
            for r in range(geo.n_expert_ranks):
                base = heap.ptrs[n_sources + r]
                side.bind_rank(r, base + lay.slab + region * SymLayout.slab_stride(geo),
                               base + lay.meta + region * SymLayout.meta_stride(geo), base + lay.dflags)
            self.sides.append(side)
        self.att = self.sides[0]                 # routes of a single-wave step live here (``norm_route`` writes them)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.layer = 0
        self.dflag_stride = n * n_sources        # dispatch flag slots per layer on an expert rank

    def _wire(self, side, tile_rows: int) -> bool:
        """E4M3 experts on decode-sized tiles take their rows quantised: half the bytes over the link and no quantise
        launch on the expert rank (``ExpertWorker._step`` makes the same call)."""
        return self.expert_format == "fp8" and wire_fp8_ok(side.geo, tile_rows)

    def begin(self, x, logits, route_kw, tile_rows=None) -> None:
        """First half of a layer's exchange: route (unless ``norm_route`` already did), plan, store the rows into the
        owners' slabs and raise their flags.  Whatever the caller launches before ``finish`` (the shared expert's GEMMs)
        runs while the expert ranks work on these rows."""
        T = x.shape[0]
        g = self.geo
        waves = g.waves(T)
        n = g.regions
        self._pending = (T, waves)
        dslot = self.layer * self.dflag_stride + self.source * n       # this source's dispatch flags of the layer
        if len(waves) == 1:
            tile_rows = tile_rows or plan_tile_rows(self.expert_format, T, g.top_k, g.num_experts)
            self.att.dispatch(x, logits, route_kw, tile_rows, dslot, self.epoch, wire_fp8=self._wire(self.att, tile_rows))
            return
        assert logits is not None, "fused routing is for single-wave steps"
        k = g.top_k
        for w, (a, b) in enumerate(waves):
            side = self.sides[w]
            side.combine = self.combine[a * k:]
            tr = plan_tile_rows(self.expert_format, b - a, k, g.num_experts)
            side.dispatch(x[a:b], logits[a:b], route_kw, tr, dslot + w, self.epoch, wire_fp8=self._wire(side, tr))

    def finish(self, out, *, shared=None, residual=None, norm_w=None, eps=0.0, x_out=None):
        """Second half: wait for every owner's completion flag and combine (slot order, + shared expert + residual,
        one rounding; optionally the next layer's input norm)."""
        T, waves = self._pending
        n = self.geo.regions
        if len(waves) == 1:
            return self.att.combine_into(out, T, self.layer * n, self.epoch, shared=shared, residual=residual, wait=True,
                                         norm_w=norm_w, eps=eps, x_out=x_out)
        for w, (a, b) in enumerate(waves):
            self.sides[w].combine_into(out[a:b], b - a, self.layer * n + w, self.epoch,
                                       shared=None if shared is None else shared[a:b],
                                       residual=None if residual is None else residual[a:b], wait=True,
                                       norm_w=norm_w, eps=eps, x_out=None if x_out is None else x_out[a:b])
        return out

    def forward(self, x, logits, route_kw, w_gate, w_up, w_down, out, *, shared=None, residual=None, tile_rows=None,
                norm_w=None, eps=0.0, x_out=None):
        self.begin(x, logits, route_kw, tile_rows)
        return self.finish(out, shared=shared, residual=residual, norm_w=norm_w, eps=eps, x_out=x_out)


CTRL_WORDS = 4 + _n.MAX_RANKS          # op, steps, reserved x2, tokens of every attention replica


class AfdAttentionEngine:
    """Wraps a single-GPU engine (GQA or MLA) whose MoE layers go through ``RemoteExchange``.  ``source`` /
    ``n_sources``: this replica's index among the data-parallel attention ranks; ``att_group``: their process group
    """

    def __init__(self, cfg: ModelConfig, weights, kv, max_tokens: int, max_seqs: int, heap: SymmetricHeap,
                 lay: SymLayout, geo: ExchangeGeometry, source: int = 0, n_sources: int = 1):
        if cfg.is_mla:
            from ..models.mla_moe import MlaMoeEngine as Engine
        else:
            from ..models.gqa_moe import GqaMoeEngine as Engine
        self.inner = Engine(cfg, weights, kv, max_tokens, max_seqs, build_moe=False)
        self.cfg, self.device = cfg, self.inner.device
        self.source, self.n_sources = source, n_sources
        # MoE layers of the main stack, then the MTP depths' decoder layers (they exchange like one more layer)
        self.moe_layers = [i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)]
        if cfg.num_experts:
            self.moe_layers += [cfg.num_layers + j for j in range(cfg.mtp_layers)]
        self.ex = RemoteExchange(geo, heap, lay, len(self.moe_layers), source, n_sources)
        self.inner.moe = self.ex
        self.inner.pre_moe = self._pre_moe
        self.ctrl = torch.zeros(CTRL_WORDS, dtype=torch.int64, device=self.device)
        self.peer_counts: list[int] | None = None     # replica 0: tokens the other replicas bring to the coming steps
        self._announced = 0
        self._replays = 0
        from .health import HealthLatch
        self.latch = HealthLatch()       # terminal: once tripped, no further step is launched against the expert ranks
        self.logits, self.next_tokens = self.inner.logits, self.inner.next_tokens

    @property
    def launches(self) -> int:
        return self.inner.launches

    @property
    def kv(self):
        return self.inner.kv

    @property
    def W(self):
        return self.inner.W

    def _pre_moe(self, layer: int) -> None:
        self.ex.layer = self.moe_layers.index(layer)

    def announce(self, T: int, steps: int, timed: bool = False, for_replay: bool = False, mtp: int = 0) -> None:
        """The next ``steps`` forward steps bring T tokens from this replica.  Replica 0 sends the message (its own T
        plus ``peer_counts`` for the other replicas; None = they bring the same number); the other replicas receive
        it here and check their own count.  ``mtp`` = j + 1 announces steps of MTP depth j alone (its decoder layer's
        exchange); 0 = steps of the main stack.  Eager calls of ``forward`` announce themselves; graph replays must
        be announced by the caller."""
        if self.source == 0:
            peers = self.peer_counts if self.peer_counts is not None else [T] * (self.n_sources - 1)
            counts = [T] + list(peers)
            assert len(counts) == self.n_sources
            self.ctrl.copy_(torch.tensor([OP_TIMED if timed else OP_STEPS, steps, mtp, 0] + counts + [0] * (_n.MAX_RANKS - len(counts)),
                                         dtype=torch.int64))
            dist.broadcast(self.ctrl, src=0)
        else:
            dist.broadcast(self.ctrl, src=0)
            words = [int(v) for v in self.ctrl.tolist()]
            if words[0] not in (OP_STEPS, OP_TIMED) or words[1] != steps or words[2] != mtp or words[4 + self.source] != T:
                raise RuntimeError(f"attention replica {self.source} expected {steps} step(s) of {T} tokens, replica 0 announced {words}")
        if not for_replay:
            self._announced += steps

    def end_round(self, active: bool = True) -> None:
        """Close a round of the script.  Replica 0 tells everybody; a replica that took part receives that message; a
        replica that sat the round out has been waiting here, answering the timing reductions of the others."""
        if self.source == 0:
            self.ctrl.copy_(torch.tensor([OP_SYNC] + [0] * (CTRL_WORDS - 1), dtype=torch.int64))
            dist.broadcast(self.ctrl, src=0)
            return
        while True:
            dist.broadcast(self.ctrl, src=0)
            op = int(self.ctrl[0].item())
            if op == OP_SYNC:
                return
            if active or op == OP_STOP:
                raise RuntimeError(f"attention replica {self.source}: unexpected control word {op} at the end of a round")
            if op == OP_TIMED:
                t = torch.zeros(1, dtype=torch.float64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)

    def announce_replays(self, T: int, steps: int) -> None:
        """Announce ``steps`` graph replays that the caller will run through ``take_replay`` (one control message
        for a whole run of decode steps instead of one per step)."""
        self.announce(T, steps, for_replay=True)
        self._replays += steps

    def take_replay(self, T: int) -> None:
        """One graph replay is about to run: covered by an earlier ``announce_replays``, or announced now."""
        if self._replays > 0:
            self._replays -= 1
        else:
            self.announce(T, 1, for_replay=True)

    def check_health(self) -> None:
        """Between steps: fold the device status word into the latch (a wait on an expert rank's flag that ran out)."""
        self.latch.check_device(K.read_status(reset=False), "attention rank")
        self.latch.require()

    def forward(self, b):
        self.latch.require()
        if not torch.cuda.is_current_stream_capturing():
            if self._announced == 0:
                self.announce(b.tokens.shape[0], 1)
            self._announced -= 1
        K.bump_epoch(self.ex.epoch)
        return self.inner.forward(b)

    def mtp_forward(self, j: int, b, next_tokens: torch.Tensor) -> torch.Tensor:
        """MTP depth j right after ``forward(b)``: its decoder layer exchanges with the expert ranks as a step of its
        own (announced here; the expert ranks then run that layer only).  Eager only.
        Reference: the drafter on the split deployment, rust/crates/cuteafd-daemon/src/shared/speculation/recurrent.rs:7-40."""
        self.latch.require()
        assert not torch.cuda.is_current_stream_capturing(), "the MTP depth of a disaggregated deployment runs eagerly"
        self.announce(b.tokens.shape[0], 1, for_replay=True, mtp=j + 1)
        K.bump_epoch(self.ex.epoch)
        return self.inner.mtp_forward(j, b, next_tokens)

    def greedy(self, logits):
        return self.inner.greedy(logits)

    def collect_max(self, ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shutdown(self) -> None:
        if self.source == 0:
            self.ctrl.copy_(torch.tensor([OP_STOP] + [0] * (CTRL_WORDS - 1), dtype=torch.int64))
        dist.broadcast(self.ctrl, src=0)


class ExpertWorker:
    """Expert-rank process: owns experts [lo, hi) of every MoE layer and serves announced steps of every attention
    replica (source).  Sources are served in rank order inside a layer; a source that sits a step out is skipped."""

    def __init__(self, cfg: ModelConfig, expert_weights: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                 heap: SymmetricHeap, lay: SymLayout, geo: ExchangeGeometry, rank: int, use_graphs: bool = True,
                 n_sources: int = 1, expert_format: str = "bf16"):
        dev = heap.buf.device
        self.cfg, self.geo, self.rank, self.er, self.n_sources = cfg, geo, rank, rank - n_sources, n_sources
        self.weights = expert_weights
        self.format = expert_format
        self.heap = heap
        self.n_layers = len(expert_weights)
        self.n_main = sum(1 for i in range(cfg.num_layers) if cfg.is_moe_layer(i))     # the rest are MTP depths' layers
        rg, n = geo.region(), geo.regions
        self.dflag_stride = n * n_sources
        flags = heap.view(lay.dflags, self.n_layers * self.dflag_stride * 4, torch.int32)
        self.sides: list[list[ExpertSide]] = []          # [source][wave]
        for a in range(n_sources):
            row = []
            for w in range(n):
                region = a * n + w
                slab = heap.view(lay.slab + region * SymLayout.slab_stride(geo), rg.max_rows * geo.hidden * 2, torch.bfloat16).view(rg.max_rows, geo.hidden)
                meta = heap.view(lay.meta + region * SymLayout.meta_stride(geo), rg.meta_ints * 4, torch.int32)
                side = ExpertSide(rg, dev, slab=slab, meta=meta, flags=flags, num_layers=self.n_layers * self.dflag_stride)
                if self.sides or row:
                    first = self.sides[0][0] if self.sides else row[0]
                    side.hbuf = first.hbuf               # the (source, wave) pairs of a step run one after the other here
                row.append(side)
            self.sides.append(row)
        self.side = self.sides[0][0]
        self.combine_ptrs = [heap.ptrs[a] + lay.combine for a in range(n_sources)]
        self.cflags_ptrs = [heap.ptrs[a] + lay.cflags for a in range(n_sources)]
        # one step counter per source: a source's flags carry its own step number
        self.epochs = [torch.zeros(1, dtype=torch.int32, device=dev) for _ in range(n_sources)]
        self.ctrl = torch.zeros(CTRL_WORDS, dtype=torch.int64, device=dev)
        self.use_graphs = use_graphs
        self.device = dev
        self.steps_served = 0

    def _step(self, counts: list[int], mtp: int = 0) -> None:
        """One announced step: the MoE layers of the main stack (``mtp`` 0) or the decoder layer of MTP depth mtp - 1."""
        g = self.geo
        n = g.regions
        lo, hi = g.rank_experts(self.er)
        active = [a for a in range(self.n_sources) if counts[a] > 0]
        for a in active:
            K.bump_epoch(self.epochs[a])
        fmt = self.format
        layers = range(min(self.n_main, self.n_layers)) if mtp == 0 else [self.n_main + mtp - 1]
        for l in layers:
            wg, wu, wd = self.weights[l]
            for a in active:
                T = counts[a]
                for w, (t0, t1) in enumerate(g.waves(T)):
                    dslot = l * self.dflag_stride + a * n + w
                    flag = self.cflags_ptrs[a] + 4 * ((l * n + w) * _n.MAX_RANKS + self.er)
                    side = self.sides[a][w]
                    combine_ptr = self.combine_ptrs[a] + t0 * g.top_k * g.hidden * 2
                    tile_rows = plan_tile_rows(fmt, t1 - t0, g.top_k, g.num_experts)
                    if fmt == "fp8":                 # E4M3 values + 128x128 block scales
                        rows = min(side.geo.max_rows, (t1 - t0) * g.top_k + (hi - lo) * tile_rows)
                        side.run_fp8(wg, wu, wd, tile_rows, rows, dslot, self.epochs[a], combine_ptr, flag, wait=True,
                                     reuse_dequant=(w > 0 or a != active[0]), wire=wire_fp8_ok(side.geo, tile_rows))
                    elif fmt in ("mxfp4", "nvfp4"):
                        side.run_w4_any(fmt, wg, wu, wd, tile_rows, dslot, self.epochs[a], combine_ptr, flag,
                                        reuse_dequant=(w > 0 or a != active[0]))
                    else:
                        side.run(wg, wu, wd, tile_rows, dslot, self.epochs[a], combine_ptr, flag, wait=True)

    def serve(self) -> None:
        while True:
            dist.broadcast(self.ctrl, src=0)
            words = [int(v) for v in self.ctrl.tolist()]
            op, steps, mtp, counts = words[0], words[1], words[2], words[4:4 + self.n_sources]
            if op == OP_STOP:
                return
            if op == OP_SYNC:
                continue
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                self._step(counts, mtp)
            b.record()
            self.steps_served += steps
            if op == OP_TIMED:
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b)], dtype=torch.float64, device=self.device)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
            st = K.read_status()
            if st:
                raise RuntimeError(f"expert rank {self.rank}: bounded wait ran out (status {st})")


def random_expert_weights(cfg: ModelConfig, lo: int, hi: int, device: torch.device, seed: int = 0, std: float = 0.02):
    g = torch.Generator(device=device).manual_seed(seed * 1000 + lo)
    out = []
    for i in range(cfg.num_layers + cfg.mtp_layers):
        if i < cfg.num_layers and not cfg.is_moe_layer(i):
            continue
        def w(*shape):
            t = torch.empty(*shape, dtype=torch.bfloat16, device=device)
            t.normal_(0.0, std, generator=g)
            return t
        out.append((w(hi - lo, cfg.expert_ffn, cfg.hidden), w(hi - lo, cfg.expert_ffn, cfg.hidden),
                    w(hi - lo, cfg.hidden, cfg.expert_ffn)))
    return out


def random_expert_weights_fp8(cfg: ModelConfig, lo: int, hi: int, device: torch.device, seed: int = 0, std: float = 0.02):
    """Random E4M3 experts with 128x128 block scales, generated and quantised on the device one layer at a time."""
    g = torch.Generator(device=device).manual_seed(seed * 1000 + lo)
    n = hi - lo

    def qw(rows: int, cols: int):
        q = torch.empty(n, rows, cols, dtype=torch.float8_e4m3fn, device=device)
        sc = torch.empty(n, rows // 128, cols // 128, dtype=torch.float32, device=device)
        for e in range(n):
            w = torch.empty(rows, cols, dtype=torch.float32, device=device).normal_(0.0, std, generator=g)
            blocks = w.view(rows // 128, 128, cols // 128, 128)
            s_ = blocks.abs().amax(dim=(1, 3)).clamp_min(1e-12) / 448.0
            q[e] = (blocks / s_[:, None, :, None]).view(rows, cols).to(torch.float8_e4m3fn)
            sc[e] = s_
        return q, sc
    out = []
    for i in range(cfg.num_layers + cfg.mtp_layers):
        if i >= cfg.num_layers or cfg.is_moe_layer(i):
            out.append((qw(cfg.expert_ffn, cfg.hidden), qw(cfg.expert_ffn, cfg.hidden), qw(cfg.hidden, cfg.expert_ffn)))
    return out


@dataclass
class AfdHandle:
    generator: object | None      # attention replicas: a Generator over the attention engine
    worker: ExpertWorker | None   # expert ranks
    parallelism: str
    replica: int = 0              # index among the attention replicas (-1 on expert ranks)
    n_replicas: int = 1

    def shutdown(self) -> None:
        if self.generator is not None:
            self.generator.engine.shutdown()

    def damaged_guards(self) -> list[str]:
        """Guard bands of this rank's exchange buffer that something wrote into (empty = every peer store stayed
        inside its region)."""
        heap = self.worker.heap if self.worker is not None else self.generator.engine.ex.heap
        return heap.damaged()


def build_afd(cfg: ModelConfig, device: torch.device, rank: int, world: int, *, max_tokens: int, max_seqs: int,
              num_pages: int, pages_per_seq: int, use_graphs: bool = True, params: dict | None = None,
              seed: int = 0, expert_format: str = "bf16", prefill_chunk: int | None = None,
              wave_tokens: int = 4096, n_attention: int = 1, snapshot: str | None = None) -> AfdHandle:
    """Create this rank's half: ranks below ``n_attention`` are data-parallel attention replicas, the others expert
    ranks.  Weights: ``snapshot`` (a checkpoint directory: the attention ranks read everything but the routed experts,
    every expert rank reads its own expert range in the stored format, nothing is re-encoded), else ``params``
    (HF-style dict of dense tensors), else random.  ``expert_format`` names the stored form of random or ``params``
    experts ("fp8" = E4M3 with 128x128 block scales, generated in that form)."""
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    A = n_attention
    assert 1 <= A < world and A <= _n.MAX_RANKS
    n_exp = world - A
    geo = ExchangeGeometry(cfg.hidden, cfg.expert_ffn, cfg.num_experts, cfg.top_k, max_tokens, n_exp,
                           wave_tokens=wave_tokens if max_tokens > wave_tokens else 0)
    n_moe = sum(1 for i in range(cfg.num_layers + cfg.mtp_layers) if (cfg.is_moe_layer(i) if i < cfg.num_layers else cfg.num_experts > 0))
    lay = SymLayout.build(geo, n_moe, A)
    heap = SymmetricHeap(lay.total, device)
    heap.arm(lay.guards(geo, A))
    torch.cuda.synchronize()
    dist.barrier()                               # nobody dispatches into a buffer whose bands are still being filled
    snap = None
    if snapshot is not None:
        from ..loader.load import expert_storage_format, open_snapshot
        snap = open_snapshot(snapshot)
        expert_format = expert_storage_format(snap)
    par = (f"afd: attention on 1 GPU + experts ep{n_exp}" if A == 1 else
           f"afd: {A} data-parallel attention replicas + experts ep{n_exp}")
    if expert_format != "bf16":
        par += f" ({expert_format} experts)"
    if rank < A:
        from ..runtime.generate import Generator
        from ..runtime.native import make_pool
        if cfg.is_mla:
            from ..models.mla_moe import LatentCache as Cache
            from ..models.mla_moe import MlaMoeWeights as Weights
        else:
            from ..models.gqa_moe import GqaMoeWeights as Weights
            from ..models.gqa_moe import KvCache as Cache
        if snap is not None:
            from ..loader.load import load_params
            _, params = load_params(snapshot, dtype=torch.bfloat16, exclude=".mlp.experts.")
        if params is not None:
            W = Weights.from_params(cfg, params, device, with_experts=False)
        else:
            W = Weights.random_init(cfg, device, seed=seed, with_experts=False)      # same seed: replicas hold the same model
        if cfg.weight_format == "fp8_block128" and cfg.is_mla:
            # an E4M3 checkpoint: decode-sized steps run q_b, the o projection and the shared expert on E4M3 twins (the
            # stored bytes when the snapshot has them, encoded once otherwise); prompt chunks keep the bf16 weights
            from ..loader.load import attach_fp8_twins
            attach_fp8_twins(W, snap, device)
        kv = Cache(cfg, num_pages, device)
        eng = AfdAttentionEngine(cfg, W, kv, max_tokens, max_seqs, heap, lay, geo, source=rank, n_sources=A)
        eng.ex.expert_format = expert_format
        gen = Generator(eng, make_pool(num_pages), pages_per_seq, max_seqs, prefill_chunk=prefill_chunk or max_tokens,
                        use_graphs=use_graphs)
        return AfdHandle(gen, None, par, rank, A)
    lo, hi = geo.rank_experts(rank - A)
    if snap is not None:
        from ..loader.load import load_experts_as_stored
        expert_format, ew = load_experts_as_stored(snap, lo, hi, device)
    elif params is not None:
        ew = []
        for i in range(cfg.num_layers + cfg.mtp_layers):
            m = f"model.layers.{i}.mlp.experts."
            if f"{m}{lo}.gate_proj.weight" not in params:
                continue
            ew.append(tuple(torch.stack([params[f"{m}{e}.{n}_proj.weight"].to(device=device, dtype=torch.bfloat16)
                                         for e in range(lo, hi)]).contiguous() for n in ("gate", "up", "down")))
        if expert_format == "fp8":       # a dense dictionary has no stored form to keep: encode once, here
            from ..quant import codecs
            ew = [tuple((torch.stack([codecs.fp8_quant_block128(w[e].float())[0] for e in range(w.shape[0])]),
                         torch.stack([codecs.fp8_quant_block128(w[e].float())[1] for e in range(w.shape[0])])) for w in trio)
                  for trio in ew]
    elif expert_format == "fp8":
        ew = random_expert_weights_fp8(cfg, lo, hi, device, seed)
    else:
        ew = random_expert_weights(cfg, lo, hi, device, seed)
    return AfdHandle(None, ExpertWorker(cfg, ew, heap, lay, geo, rank, use_graphs, n_sources=A, expert_format=expert_format),
                     par, -1, A)
