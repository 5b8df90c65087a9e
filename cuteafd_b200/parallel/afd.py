"""Attention/FFN disaggregation over one NVLink domain: rank 0 runs the backbone (attention,
router, head, KV cache); ranks 1..N-1 hold the routed experts, partitioned by expert id.

Data path (no NCCL, no host hop): every rank maps one symmetric buffer of every other rank
(``torch.distributed._symmetric_memory`` does the handle exchange).  The attention rank's plan and
dispatch kernels store tile lists and token rows straight into the owners' buffers and publish a
per-layer step number; the owners' grouped tcgen05 GEMMs wait for it, and the fc2 epilogue stores
each (token, slot) row straight into the attention rank's combine buffer and publishes the step
number back; the combine kernel waits for every owner.  Kernel waits are bounded and report
through the status word.

Control path: one small NCCL broadcast per forward call (op, tokens, steps) so expert ranks know
how many layer sequences to launch; a run of decode steps is announced once and then proceeds on
device flags only.

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
from .moe_exchange import AttentionSide, ExchangeGeometry, ExpertSide, pick_tile_rows

OP_STOP, OP_STEPS, OP_TIMED = 0, 1, 2


def _align(x: int, a: int = 1024) -> int:
    return (x + a - 1) // a * a


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
    def build(geo: ExchangeGeometry, num_layers: int) -> "SymLayout":
        """``geo.regions`` slab regions and plan blocks (one per wave of a large step) and one flag slot per
        (layer, region); slot = layer * regions + region."""
        rg, n = geo.region(), geo.regions
        o = 0
        slab = o; o = _align(o + n * SymLayout.slab_stride(geo))
        meta = o; o = _align(o + n * SymLayout.meta_stride(geo))
        dflags = o; o = _align(o + num_layers * n * 4)
        combine = o; o = _align(o + geo.max_tokens * geo.top_k * geo.hidden * 2)
        cflags = o; o = _align(o + num_layers * n * _n.MAX_RANKS * 4)
        return SymLayout(slab, meta, dflags, combine, cflags, o)

    @staticmethod
    def slab_stride(geo: ExchangeGeometry) -> int:
        return _align(geo.region().max_rows * geo.hidden * 2)

    @staticmethod
    def meta_stride(geo: ExchangeGeometry) -> int:
        return _align(geo.region().meta_ints * 4)


class SymmetricHeap:
    def __init__(self, nbytes: int, device: torch.device, group=None):
        import torch.distributed._symmetric_memory as symm_mem
        group = group or dist.group.WORLD
        try:
            symm_mem.enable_symm_mem_for_group(group.group_name)
        except Exception:
            pass
        self.buf = symm_mem.empty(nbytes, dtype=torch.uint8, device=device)
        self.buf.zero_()
        self.handle = symm_mem.rendezvous(self.buf, group)
        self.ptrs = [int(p) for p in self.handle.buffer_ptrs]
        torch.cuda.synchronize()
        dist.barrier()

    def view(self, offset: int, nbytes: int, dtype: torch.dtype) -> torch.Tensor:
        return self.buf[offset:offset + nbytes].view(dtype)


class RemoteExchange:
    """Attention-rank half: same interface as ``LocalExchange`` with experts on other GPUs.  A step larger than
    ``geo.wave_tokens`` goes out as several waves (own slab region / plan block / flags each)."""

    def __init__(self, geo: ExchangeGeometry, heap: SymmetricHeap, lay: SymLayout, num_layers: int, rank: int):
        dev = heap.buf.device
        self.geo, self.heap, self.lay = geo, heap, lay
        rg, n = geo.region(), geo.regions
        self.combine = heap.view(lay.combine, geo.max_tokens * geo.top_k * geo.hidden * 2, torch.bfloat16).view(-1, geo.hidden)
        cflags = heap.view(lay.cflags, num_layers * n * _n.MAX_RANKS * 4, torch.int32)
        self.sides: list[AttentionSide] = []
        for w in range(n):
            side = AttentionSide(rg, dev, combine=self.combine, flags=cflags, num_layers=num_layers * n)
            for r in range(geo.n_expert_ranks):
                base = heap.ptrs[1 + r]
                side.bind_rank(r, base + lay.slab + w * SymLayout.slab_stride(geo), base + lay.meta + w * SymLayout.meta_stride(geo),
                               base + lay.dflags)
            self.sides.append(side)
        self.att = self.sides[0]                 # routes of a single-wave step live here (``norm_route`` writes them)
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.layer = 0

    def forward(self, x, logits, route_kw, w_gate, w_up, w_down, out, *, shared=None, residual=None, tile_rows=None,
                norm_w=None, eps=0.0, x_out=None):
        T = x.shape[0]
        g = self.geo
        waves = g.waves(T)
        n = g.regions
        if len(waves) == 1:
            tile_rows = tile_rows or pick_tile_rows(T, g.top_k, g.num_experts)
            self.att.dispatch(x, logits, route_kw, tile_rows, self.layer * n, self.epoch)
            return self.att.combine_into(out, T, self.layer * n, self.epoch, shared=shared, residual=residual, wait=True,
                                         norm_w=norm_w, eps=eps, x_out=x_out)
        assert logits is not None, "fused routing is for single-wave steps"
        k = g.top_k
        for w, (a, b) in enumerate(waves):
            side = self.sides[w]
            side.combine = self.combine[a * k:]
            side.dispatch(x[a:b], logits[a:b], route_kw, pick_tile_rows(b - a, k, g.num_experts), self.layer * n + w, self.epoch)
        for w, (a, b) in enumerate(waves):
            self.sides[w].combine_into(out[a:b], b - a, self.layer * n + w, self.epoch,
                                       shared=None if shared is None else shared[a:b],
                                       residual=None if residual is None else residual[a:b], wait=True,
                                       norm_w=norm_w, eps=eps, x_out=None if x_out is None else x_out[a:b])
        return out


class AfdAttentionEngine:
    """Wraps a single-GPU engine (GQA or MLA) whose MoE layers go through ``RemoteExchange``."""

    def __init__(self, cfg: ModelConfig, weights, kv, max_tokens: int, max_seqs: int, heap: SymmetricHeap,
                 lay: SymLayout, geo: ExchangeGeometry):
        if cfg.is_mla:
            from ..models.mla_moe import MlaMoeEngine as Engine
        else:
            from ..models.gqa_moe import GqaMoeEngine as Engine
        self.inner = Engine(cfg, weights, kv, max_tokens, max_seqs, build_moe=False)
        self.cfg, self.device = cfg, self.inner.device
        self.moe_layers = [i for i in range(cfg.num_layers) if cfg.is_moe_layer(i)]
        self.ex = RemoteExchange(geo, heap, lay, len(self.moe_layers), 0)
        self.inner.moe = self.ex
        self.inner.pre_moe = self._pre_moe
        self.ctrl = torch.zeros(4, dtype=torch.int64, device=self.device)
        self._announced = 0
        from .health import HealthLatch
        self.latch = HealthLatch()       # terminal: once tripped, no further step is launched against the expert ranks
        self.logits, self.next_tokens = self.inner.logits, self.inner.next_tokens

    @property
    def launches(self) -> int:
        return self.inner.launches

    def _pre_moe(self, layer: int) -> None:
        self.ex.layer = self.moe_layers.index(layer)

    def announce(self, T: int, steps: int, timed: bool = False, for_replay: bool = False) -> None:
        """Tell the expert ranks how many forward steps follow (each with T tokens).  Eager calls of
        ``forward`` announce themselves; graph replays must be announced by the caller."""
        self.ctrl.copy_(torch.tensor([OP_TIMED if timed else OP_STEPS, T, steps, 0], dtype=torch.int64))
        dist.broadcast(self.ctrl, src=0)
        if not for_replay:
            self._announced += steps

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

    def greedy(self, logits):
        return self.inner.greedy(logits)

    def collect_max(self, ms: float) -> float:
        t = torch.tensor([ms], dtype=torch.float64, device=self.device)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    def shutdown(self) -> None:
        self.ctrl.copy_(torch.tensor([OP_STOP, 0, 0, 0], dtype=torch.int64))
        dist.broadcast(self.ctrl, src=0)


class ExpertWorker:
    """Expert-rank process: owns experts [lo, hi) of every MoE layer and serves announced steps."""

    def __init__(self, cfg: ModelConfig, expert_weights: list[tuple[torch.Tensor, torch.Tensor, torch.Tensor]],
                 heap: SymmetricHeap, lay: SymLayout, geo: ExchangeGeometry, rank: int, use_graphs: bool = True):
        dev = heap.buf.device
        self.cfg, self.geo, self.rank, self.er = cfg, geo, rank, rank - 1
        self.weights = expert_weights
        self.n_layers = len(expert_weights)
        rg, n = geo.region(), geo.regions
        flags = heap.view(lay.dflags, self.n_layers * n * 4, torch.int32)
        self.sides: list[ExpertSide] = []
        for w in range(n):
            slab = heap.view(lay.slab + w * SymLayout.slab_stride(geo), rg.max_rows * geo.hidden * 2, torch.bfloat16).view(rg.max_rows, geo.hidden)
            meta = heap.view(lay.meta + w * SymLayout.meta_stride(geo), rg.meta_ints * 4, torch.int32)
            side = ExpertSide(rg, dev, slab=slab, meta=meta, flags=flags, num_layers=self.n_layers * n)
            if w:
                side.hbuf = self.sides[0].hbuf           # the waves of a step run one after the other on this rank
            self.sides.append(side)
        self.side = self.sides[0]
        self.combine_ptr = heap.ptrs[0] + lay.combine
        self.cflags_ptr = heap.ptrs[0] + lay.cflags
        self.epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        self.ctrl = torch.zeros(4, dtype=torch.int64, device=dev)
        self.use_graphs = use_graphs
        self.graphs: dict[int, torch.cuda.CUDAGraph] = {}
        self.device = dev
        self.steps_served = 0

    def _step(self, T: int) -> None:
        K.bump_epoch(self.epoch)
        g = self.geo
        n = g.regions
        lo, hi = g.rank_experts(self.er)
        waves = g.waves(T)
        fp8 = bool(self.weights) and isinstance(self.weights[0][0], tuple)
        for l, (wg, wu, wd) in enumerate(self.weights):
            for w, (a, b) in enumerate(waves):
                slot = l * n + w
                flag = self.cflags_ptr + 4 * (slot * _n.MAX_RANKS + self.er)
                side = self.sides[w]
                combine_ptr = self.combine_ptr + a * g.top_k * g.hidden * 2
                tile_rows = pick_tile_rows(b - a, g.top_k, g.num_experts)
                if fp8:                          # E4M3 values + 128x128 block scales
                    if tile_rows == 128 and (b - a) * g.top_k < 64 * g.num_experts:
                        tile_rows = 64           # the fp8 kernel's weights-on-M path tops out at 64 rows
                    rows = min(side.geo.max_rows, (b - a) * g.top_k + (hi - lo) * tile_rows)
                    side.run_fp8(wg, wu, wd, tile_rows, rows, slot, self.epoch, combine_ptr, flag, wait=True,
                                 reuse_dequant=w > 0)
                else:
                    side.run(wg, wu, wd, tile_rows, slot, self.epoch, combine_ptr, flag, wait=True)

    def serve(self) -> None:
        g = self.geo
        while True:
            dist.broadcast(self.ctrl, src=0)
            op, T, steps, _ = (int(v) for v in self.ctrl.tolist())
            if op == OP_STOP:
                return
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            a.record()
            for _ in range(steps):
                self._step(T)
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
    for i in range(cfg.num_layers):
        if not cfg.is_moe_layer(i):
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
    for i in range(cfg.num_layers):
        if cfg.is_moe_layer(i):
            out.append((qw(cfg.expert_ffn, cfg.hidden), qw(cfg.expert_ffn, cfg.hidden), qw(cfg.hidden, cfg.expert_ffn)))
    return out


@dataclass
class AfdHandle:
    generator: object | None      # rank 0: a Generator over the attention engine
    worker: ExpertWorker | None   # other ranks
    parallelism: str

    def shutdown(self) -> None:
        if self.generator is not None:
            self.generator.engine.shutdown()


def build_afd(cfg: ModelConfig, device: torch.device, rank: int, world: int, *, max_tokens: int, max_seqs: int,
              num_pages: int, pages_per_seq: int, use_graphs: bool = True, params: dict | None = None,
              seed: int = 0, expert_format: str = "bf16", prefill_chunk: int | None = None,
              wave_tokens: int = 4096) -> AfdHandle:
    """Create this rank's half.  ``params`` (HF-style dict) gives real weights; otherwise random.
    ``expert_format`` "fp8" keeps the routed experts as E4M3 with 128x128 block scales on the expert ranks."""
    os.environ.setdefault("CUDA_MODULE_LOADING", "EAGER")
    n_exp = world - 1
    geo = ExchangeGeometry(cfg.hidden, cfg.expert_ffn, cfg.num_experts, cfg.top_k, max_tokens, n_exp,
                           wave_tokens=wave_tokens if max_tokens > wave_tokens else 0)
    n_moe = sum(1 for i in range(cfg.num_layers) if cfg.is_moe_layer(i))
    lay = SymLayout.build(geo, n_moe)
    heap = SymmetricHeap(lay.total, device)
    par = f"afd: attention on 1 GPU + experts ep{n_exp}"
    if expert_format != "bf16":
        par += f" ({expert_format} experts)"
    if rank == 0:
        from ..runtime.generate import Generator
        from ..runtime.paged import PagePool
        if cfg.is_mla:
            from ..models.mla_moe import LatentCache as Cache
            from ..models.mla_moe import MlaMoeWeights as Weights
        else:
            from ..models.gqa_moe import GqaMoeWeights as Weights
            from ..models.gqa_moe import KvCache as Cache
        if params is not None:
            W = Weights.from_params(cfg, params, device, with_experts=False)
        else:
            W = Weights.random_init(cfg, device, seed=seed, with_experts=False)
        kv = Cache(cfg, num_pages, device)
        eng = AfdAttentionEngine(cfg, W, kv, max_tokens, max_seqs, heap, lay, geo)
        gen = Generator(eng, PagePool(num_pages), pages_per_seq, max_seqs, prefill_chunk=prefill_chunk or max_tokens,
                        use_graphs=use_graphs)
        return AfdHandle(gen, None, par)
    lo, hi = geo.rank_experts(rank - 1)
    if params is not None:
        ew = []
        for i in range(cfg.num_layers):
            if not cfg.is_moe_layer(i):
                continue
            m = f"model.layers.{i}.mlp.experts."
            ew.append(tuple(torch.stack([params[f"{m}{e}.{n}_proj.weight"].to(device=device, dtype=torch.bfloat16)
                                         for e in range(lo, hi)]).contiguous() for n in ("gate", "up", "down")))
        if expert_format == "fp8":
            from ..quant import codecs
            ew = [tuple((torch.stack([codecs.fp8_quant_block128(w[e].float())[0] for e in range(w.shape[0])]),
                         torch.stack([codecs.fp8_quant_block128(w[e].float())[1] for e in range(w.shape[0])])) for w in trio)
                  for trio in ew]
    elif expert_format == "fp8":
        ew = random_expert_weights_fp8(cfg, lo, hi, device, seed)
    else:
        ew = random_expert_weights(cfg, lo, hi, device, seed)
    return AfdHandle(None, ExpertWorker(cfg, ew, heap, lay, geo, rank, use_graphs), par)
