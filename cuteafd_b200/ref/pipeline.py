"""The oracle decoder run as pipeline stages: stage s owns the layers ``plan.layers(s)`` (and their K/V), the first
stage embeds, the last applies the head, and the residual stream crosses every boundary through a ``Hop``.  This is the
CPU twin of a pipeline-parallel engine: the same stage plan and the same hop object that ``parallel/pp.py`` gives the
GPUs, with gloo ranks instead.  Counterpart: the layer-range placement of the reference
(rust/crates/cuteafd-loader/src/placement/attention.rs:5-45) and its hop executor (peer_split/hop.rs).
"""
from __future__ import annotations

import torch

from ..parallel.pp import Hop, StagePlan
from .model import KvState, RefDecoder


class PipelinedDecoder:
    def __init__(self, decoder: RefDecoder, plan: StagePlan, stage: int, group=None):
        self.dec, self.plan, self.stage = decoder, plan, stage
        self.stages = len(plan.bounds) - 1
        self.prev = Hop(stage - 1, group) if stage > 0 else None
        self.next = Hop(stage + 1, group) if stage < self.stages - 1 else None

    def forward(self, tokens: torch.Tensor, kv: KvState) -> torch.Tensor | None:
        """Append ``tokens``; returns the logits [T, vocab] on the last stage, None on the others."""
        own = self.plan.layers(self.stage)
        start = kv.length(own[0]) if len(own) else 0
        T = tokens.shape[0]
        positions = torch.arange(start, start + T)
        if self.stage == 0:
            h = self.dec.embed(tokens)
        else:
            like = self.dec.embed(tokens[:1])
            h = self.prev.recv(torch.empty(T, like.shape[1], dtype=like.dtype))
        for i in own:
            h = self.dec.layer(i, h, positions, kv)
        if self.next is not None:
            self.next.send(h)
            return None
        return self.dec.head(h)
