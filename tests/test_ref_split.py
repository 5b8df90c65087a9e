"""Tiny MoE decoder: whole run versus 1 attention rank + 2 expert ranks over gloo."""
import torch

from cuteafd_b200 import tiny_moe
from cuteafd_b200.ref import split


def test_whole_vs_split_logits_match():
    cfg = tiny_moe()
    prompts = split.tiny_prompts(cfg, batch=2, length=64, seed=1)
    wt, wl = split.run_whole(cfg, prompts, steps=16)
    st, sl = split.run_split(cfg, prompts, steps=16, expert_ranks=2)
    assert torch.equal(wt, st)
    assert torch.equal(wl, sl), (wl - sl).abs().max()


def test_expert_range_covers_all():
    for n, r in ((128, 7), (256, 6), (8, 2), (128, 3)):
        spans = [split.expert_range(n, r, i) for i in range(r)]
        assert spans[0][0] == 0 and spans[-1][1] == n
        assert all(a[1] == b[0] for a, b in zip(spans, spans[1:]))
