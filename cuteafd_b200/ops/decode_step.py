"""Front end of the one-launch decode step (``csrc/decode_step.cu``): the per-layer pointer table, the argument
block, the workspaces and the launch.

A decode step of at most 32 rows (one new token per sequence) of a GQA + MoE decoder can run as one persistent
cooperative kernel instead of ~10 launches per layer.  It is opt-in (``CAFD_FUSED_DECODE=1``): measured on a B200 with
the Qwen3-30B-A3B shape it takes 125 / 294 us per layer at 1 / 8 rows against 102 / 199 us for the per-op tcgen05
kernels, because with one 8-warp CTA per SM its mma.sync inner loops are bound by instruction issue, not by HBM.
``FusedDecodeStep.supports(cfg)`` says which geometries it takes; everything else (prefill, verify rows, shared
experts, dense layers) stays on the per-op kernels.  The
reference replays one CUDA graph segment per layer (rust/crates/cuteafd-daemon/src/families/glm5/engine.rs:2208-2210);
this is the same step with the kernel boundaries removed.
"""
from __future__ import annotations

import ctypes as C
import math
import os

import torch

from .._native import lib as _n
from . import kernels as K

MAX_RANKS = 8
MAX_ENTRIES = 1024
_P = C.c_void_p


class DecodeLayer(C.Structure):
    _fields_ = [(n, _P) for n in ("ln1", "ln2", "wqkv", "wo", "q_norm", "k_norm", "router", "router_bias", "w_gate", "w_up",
                                  "w_down", "k_cache", "v_cache")]


class DecodeArgs(C.Structure):
    _fields_ = ([(n, _P) for n in ("layers", "embed", "final_norm", "lm_head", "inv_freq", "tokens", "positions", "slots",
                                   "seq_lens", "page_table", "h", "qkv", "attn", "rlogits", "hbuf", "cbuf", "part", "rope_cs", "tickets",
                                   "logits", "next_tokens", "cand_v", "cand_i", "bar", "status")]
                + [(n, _P * MAX_RANKS) for n in ("slab", "meta", "dflag", "cbuf_of", "cflag")]
                + [("epoch", _P), ("trace", _P)]
                + [(n, C.c_int) for n in ("n_ranks", "my_rank", "slab_rows", "num_layers", "T", "max_pages", "splits", "H", "Hq",
                                          "Hkv", "E", "top_k", "I", "V", "ld_logits", "rope_interleaved", "sigmoid", "num_groups",
                                          "topk_groups", "normalize", "advance", "ring_stages")]
                + [(n, C.c_float) for n in ("eps", "routed_scale", "scale_log2")])


def _lib():
    L = _n.cuda_lib()
    if not getattr(L, "_decode_step_sigs", False):
        L.cafd_decode_step.argtypes = [C.c_void_p, C.c_int, C.c_void_p]
        L.cafd_decode_step.restype = C.c_int
        for name in ("cafd_decode_step_layer_bytes", "cafd_decode_step_args_bytes", "cafd_decode_step_max_rows"):
            getattr(L, name).argtypes = []
            getattr(L, name).restype = C.c_int
        L.cafd_decode_step_part_floats.argtypes = [C.c_int, C.c_int, C.c_int]
        L.cafd_decode_step_part_floats.restype = C.c_longlong
        assert L.cafd_decode_step_layer_bytes() == C.sizeof(DecodeLayer), "DecodeLayer layout differs from the library's"
        assert L.cafd_decode_step_args_bytes() == C.sizeof(DecodeArgs), "DecodeArgs layout differs from the library's"
        L._decode_step_sigs = True
    return L


def pick_splits(rows: int, kv_heads: int, max_pages: int, num_sms: int) -> int:
    """KV splits per (sequence, kv head): the items are spread over 2 x SMs four-warp groups; cost of a choice =
    rounds of items per group x (pages per item + a fixed part for the query set-up) + the merge over the splits."""
    slots = 2 * num_sms
    best, best_cost = 1, None
    for s in range(1, min(64, max(1, max_pages)) + 1):
        rounds = -(-rows * kv_heads * s // slots)
        cost = rounds * (-(-max_pages // s) + 3) + 0.25 * s
        if best_cost is None or cost < best_cost:
            best, best_cost = s, cost
    return best


class FusedDecodeStep:
    """Workspaces + argument block of the one-launch decode step for one engine."""
    MAX_ROWS = 32

    @staticmethod
    def supports(cfg) -> bool:
        if os.environ.get("CAFD_FUSED_DECODE", "0") != "1":
            return False
        return (cfg.attention == "gqa" and cfg.head_dim == 128 and cfg.hidden <= 2048 and cfg.hidden % 256 == 0
                and 0 < cfg.num_experts <= 256 and cfg.top_k <= 8 and cfg.expert_ffn % 256 == 0 and not cfg.num_shared_experts
                and cfg.first_dense_layers == 0 and all(cfg.is_moe_layer(i) for i in range(cfg.num_layers))
                and (cfg.num_heads * 128) % 256 == 0 and cfg.num_heads % cfg.num_kv_heads == 0
                and cfg.num_heads // cfg.num_kv_heads <= 16 and cfg.num_groups <= 32
                and not cfg.attention_bias and cfg.rope_dim == cfg.head_dim and not cfg.sliding_window)

    def __init__(self, engine):
        cfg, W, dev = engine.cfg, engine.W, engine.device
        self.engine, self.cfg, self.device = engine, cfg, dev
        L = _lib()
        self.lib = L
        # ---- per-layer pointer table (device copy kept alive here) ----
        tbl = (DecodeLayer * cfg.num_layers)()
        for i in range(cfg.num_layers):
            lw = W.layers[i]
            t = tbl[i]
            t.ln1, t.ln2, t.wqkv, t.wo = lw.ln1.data_ptr(), lw.ln2.data_ptr(), lw.wqkv.data_ptr(), lw.wo.data_ptr()
            t.q_norm = lw.q_norm.data_ptr() if lw.q_norm is not None else None
            t.k_norm = lw.k_norm.data_ptr() if lw.k_norm is not None else None
            t.router = lw.router.data_ptr()
            t.router_bias = lw.router_bias.data_ptr() if lw.router_bias is not None else None
            t.w_gate, t.w_up, t.w_down = lw.w_gate.data_ptr(), lw.w_up.data_ptr(), lw.w_down.data_ptr()
            t.k_cache, t.v_cache = engine.kv.k[i].data_ptr(), engine.kv.v[i].data_ptr()
        raw = bytes(tbl)
        self.layer_table = torch.frombuffer(bytearray(raw), dtype=torch.uint8).to(dev)
        n = self.MAX_ROWS
        self.hbuf = torch.empty(MAX_ENTRIES, cfg.expert_ffn, dtype=torch.bfloat16, device=dev)
        self.cbuf = torch.empty(n * cfg.top_k, cfg.hidden, dtype=torch.bfloat16, device=dev)
        self.sync = torch.zeros(64 + n * cfg.num_kv_heads, dtype=torch.int32, device=dev)      # [0] arrivals [1] abort; tickets from 64
        self.sms = K.num_sms()
        self.cand_v = torch.empty(self.sms * 32, dtype=torch.float32, device=dev)
        self.cand_i = torch.empty(self.sms * 32, dtype=torch.int32, device=dev)
        self.part: torch.Tensor | None = None
        self.rlogits = torch.empty(n, cfg.num_experts, dtype=torch.float32, device=dev)
        self.rope_cs = torch.empty(n, 64, 2, dtype=torch.float32, device=dev)
        self.launches = 0
        self.trace: torch.Tensor | None = None      # int64 [phases + 1]: set to record CTA 0's clock after every barrier

    def run(self, b, advance: bool = False) -> tuple[torch.Tensor, torch.Tensor]:
        """One step over batch ``b`` (one new token per sequence).  Returns (fp32 logits [T, vocab], next tokens [T])."""
        eng, cfg = self.engine, self.cfg
        T = b.tokens.shape[0]
        S, max_pages = b.page_table.shape
        assert S == T and T <= self.MAX_ROWS and not b.prefill and b.max_q_len == 1
        splits = pick_splits(T, cfg.num_kv_heads, max_pages, self.sms)
        need = int(self.lib.cafd_decode_step_part_floats(T, cfg.num_kv_heads, splits))
        if self.part is None or self.part.numel() < need:
            assert not torch.cuda.is_current_stream_capturing(), "the split-KV scratch must exist before capture"
            self.part = torch.empty(need, dtype=torch.float32, device=self.device)
        ws = eng.ws
        a = DecodeArgs()
        a.layers = self.layer_table.data_ptr()
        a.embed, a.final_norm, a.lm_head = eng.W.embed.data_ptr(), eng.W.final_norm.data_ptr(), eng.W.lm_head.data_ptr()
        a.inv_freq = eng.inv_freq.data_ptr()
        a.tokens, a.positions, a.slots = b.tokens.data_ptr(), b.positions.data_ptr(), b.slots.data_ptr()
        a.seq_lens, a.page_table = b.seq_lens.data_ptr(), b.page_table.data_ptr()
        a.h, a.qkv, a.attn = ws.h.data_ptr(), ws.qkv.data_ptr(), ws.attn.data_ptr()
        a.rlogits, a.hbuf, a.cbuf = self.rlogits.data_ptr(), self.hbuf.data_ptr(), self.cbuf.data_ptr()
        a.part, a.tickets = self.part.data_ptr(), self.sync.data_ptr() + 64 * 4
        a.rope_cs = self.rope_cs.data_ptr()
        a.logits, a.next_tokens = eng.logits.data_ptr(), eng.next_tokens.data_ptr()
        a.cand_v, a.cand_i = self.cand_v.data_ptr(), self.cand_i.data_ptr()
        a.bar, a.status = self.sync.data_ptr(), K.status_word(self.device).data_ptr()
        a.trace = self.trace.data_ptr() if self.trace is not None else None
        a.n_ranks, a.my_rank, a.slab_rows = 1, 0, 0
        a.num_layers, a.T, a.max_pages, a.splits = cfg.num_layers, T, max_pages, splits
        a.H, a.Hq, a.Hkv, a.E, a.top_k, a.I, a.V = (cfg.hidden, cfg.num_heads, cfg.num_kv_heads, cfg.num_experts, cfg.top_k,
                                                     cfg.expert_ffn, cfg.vocab_size)
        a.ld_logits = eng.logits.stride(0)
        a.rope_interleaved, a.sigmoid = int(cfg.rope_interleaved), int(cfg.scoring == "sigmoid")
        a.num_groups, a.topk_groups, a.normalize = cfg.num_groups, cfg.topk_groups, int(cfg.norm_topk_prob)
        a.advance = int(advance)
        a.eps, a.routed_scale = cfg.rms_eps, cfg.routed_scale
        a.scale_log2 = (1.0 / math.sqrt(cfg.head_dim)) * 1.4426950408889634
        _n.check(self.lib.cafd_decode_step(C.byref(a), self.sms, K._stream()), "cafd_decode_step")
        self.launches += 1
        return eng.logits[:T], eng.next_tokens[:T]
