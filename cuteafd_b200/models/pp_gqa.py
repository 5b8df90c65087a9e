"""Pipeline stages for the GQA MoE family: stage s of a ``StagePlan`` owns a contiguous range of decoder layers with
their weights and their K/V pages, the first stage embeds, the last applies the final norm and the head, and the
residual stream of a step crosses each boundary once through a ``Hop`` (NCCL point-to-point on a side stream).

Every stage is driven with the same batches (token ids, positions, page tables are tiny and already on every rank's
device); only the [T, hidden] residual rows move.  The selected tokens go back from the last stage to the others in one
4-byte-per-row broadcast, so a ``Generator`` on every rank advances in lockstep.  Several micro-batches in flight keep
all stages busy: ``forward_micro`` posts stage s's receive of micro-batch m + 1 while it still computes micro-batch m.

Reference: layer-range placement (rust/crates/cuteafd-loader/src/placement/attention.rs:5-45), residual hop points
(rust/crates/cuteafd-loader/src/placement/residual.rs:62-71) and the hop executor
(rust/crates/cuteafd-daemon/src/shared/peer_split/hop.rs).
"""
from __future__ import annotations

import torch
import torch.distributed as dist

from ..config import ModelConfig
from ..ops import kernels as K
from ..parallel.pp import RingHop, StagePlan
from .gqa_moe import Batch, GqaMoeEngine, GqaMoeWeights, KvCache


def stage_config(cfg: ModelConfig, plan: StagePlan, stage: int) -> ModelConfig:
    """The model a stage sees: its own layers only, renumbered from 0 (dense-prefix layers that fall into the range
    stay dense), no MTP depth (that belongs to the last stage's drafter, not to the stack)."""
    own = plan.layers(stage)
    dense = max(0, min(len(own), cfg.first_dense_layers - own.start))
    return cfg.replace(num_layers=len(own), first_dense_layers=dense, mtp_layers=0,
                       window_layers=tuple(cfg.window_layers[own.start:own.stop]))


def stage_params(cfg: ModelConfig, params: dict, plan: StagePlan, stage: int) -> dict:
    """Name -> tensor dictionary of one stage: ``model.layers.{i}`` of its range renumbered from 0, plus the embedding
    (first stage reads it) and the final norm / head (last stage reads them)."""
    own = plan.layers(stage)
    out = {}
    for name, t in params.items():
        if name.startswith("model.layers."):
            i, rest = name[len("model.layers."):].split(".", 1)
            if int(i) in own:
                out[f"model.layers.{int(i) - own.start}.{rest}"] = t
        else:
            out[name] = t
    return out


class PpGqaMoeEngine(GqaMoeEngine):
    """One pipeline stage.  ``forward`` returns the logits on the last stage and None elsewhere; ``greedy`` returns the
    selected tokens on every stage."""

    def __init__(self, cfg: ModelConfig, params: dict, plan: StagePlan, stage: int, num_pages: int, max_tokens: int,
                 max_seqs: int = 64, group=None, device: torch.device | None = None):
        self.group = group or dist.group.WORLD
        self.plan, self.stage, self.stages = plan, stage, len(plan.bounds) - 1
        assert dist.get_world_size(self.group) == self.stages and dist.get_rank(self.group) == stage
        dev = device or torch.device("cuda", torch.cuda.current_device())
        local = stage_config(cfg, plan, stage)
        W = GqaMoeWeights.from_params(local, stage_params(cfg, params, plan, stage), dev)
        super().__init__(local, W, KvCache(local, num_pages, dev), max_tokens, max_seqs)
        self.full_cfg = cfg
        self.first, self.last = stage == 0, stage == self.stages - 1
        ring = dict(rows=max_tokens, width=cfg.hidden)
        self.prev = RingHop(stage - 1, self.group, dev, **ring) if not self.first else None
        self.next = RingHop(stage + 1, self.group, dev, **ring) if not self.last else None
        self._rows = 0
        self.hops = 0

    def _layers(self, T: int, b: Batch) -> None:
        cfg, ws = self.cfg, self.ws
        have_x = False
        for i in range(cfg.num_layers):
            L = self.W.layers[i]
            if not have_x:
                K.rmsnorm(ws.h[:T], L.ln1, cfg.rms_eps, out=ws.x[:T])
                self.launches += 1
            self._attention(i, T, b)
            nxt = self.W.layers[i + 1].ln1 if i + 1 < cfg.num_layers else None
            have_x = self._ffn(i, T, nxt)

    def forward(self, b: Batch) -> torch.Tensor | None:
        cfg, ws = self.cfg, self.ws
        T = b.tokens.shape[0]
        assert T <= self.max_tokens
        self._rows = int(b.last_rows.shape[0]) if b.last_rows is not None else T
        if self.first:
            K.embed(b.tokens, self.W.embed, out=ws.h[:T])
            self.launches += 1
            if b.embeds is not None:
                ws.h[:T].index_copy_(0, b.embeds[0], b.embeds[1])
        else:
            self.prev.recv(ws.h[:T])
            self.hops += 1
        self._layers(T, b)
        if not self.last:
            self.next.send(ws.h[:T])
            self.hops += 1
            return None
        rows = ws.h[:T].index_select(0, b.last_rows) if b.last_rows is not None else ws.h[:T]
        n = rows.shape[0]
        xn = K.rmsnorm(rows, self.W.final_norm, cfg.rms_eps, out=ws.x[:n])
        logits = K.linear(xn, self.W.lm_head, out=self.logits[:n], out_f32=True)
        self.launches += 2
        return logits

    def select(self, logits: torch.Tensor | None, out: torch.Tensor | None = None) -> torch.Tensor:
        """Last stage: argmax of the step's logits into ``out`` (default: the engine's token buffer); the other stages
        only name the buffer the tokens will be received into."""
        out = self.next_tokens[:self._rows] if out is None else out
        if self.last:
            K.argmax(logits, out=out)
            self.launches += 1
        return out

    def share(self, tokens: torch.Tensor) -> torch.Tensor:
        """The last stage's selection on every stage (4 bytes per row)."""
        dist.broadcast(tokens, src=dist.get_global_rank(self.group, self.stages - 1), group=self.group)
        return tokens

    def greedy(self, logits: torch.Tensor | None) -> torch.Tensor:
        """Tokens of the last ``forward`` on every stage (``logits`` is None on all but the last)."""
        return self.share(self.select(logits))

    def forward_micro(self, batches: list[Batch]) -> list[torch.Tensor]:
        """Independent micro-batches through the pipeline; returns their tokens on every stage.  All forwards are
        enqueued before any token comes back, so stage s works on micro-batch m while stage s + 1 works on m - 1 and
        the hops (staged through their own ring on side streams) overlap both."""
        picks = []
        for b in batches:
            logits = self.forward(b)
            picks.append(self.select(logits, torch.empty(self._rows, dtype=torch.int32, device=self.device)))
        return [self.share(t) for t in picks]
