"""Context split over gloo CPU ranks: page-parity KV partition, query all-gather, partial attention + LSE merge and
the indexer's candidate merge against whole-sequence attention."""
import os
import socket

import torch

from cuteafd_b200.parallel import context_split as CS
from cuteafd_b200.ref import ops as R


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def test_merge_is_exact_on_one_process():
    g = torch.Generator().manual_seed(0)
    Tk, Tq, H, Hk, D = 300, 5, 8, 2, 32
    q, k, v = torch.randn(Tq, H, D, generator=g), torch.randn(Tk, Hk, D, generator=g), torch.randn(Tk, Hk, D, generator=g)
    start = Tk - Tq
    want = R.causal_attention(q, k, v, start).float()
    q_pos = torch.arange(start, Tk)
    for ranks in (2, 3):
        parts = []
        for r in range(ranks):
            pos = CS.local_positions(Tk, r, ranks)
            parts.append(CS.partial_attention(q, k[pos], v[pos], pos, q_pos, 1.0 / D ** 0.5))
        assert torch.allclose(CS.merge_partials(parts), want, atol=1e-5)
    # a row that sees nothing on one rank (short sequence: only page 0 exists) merges cleanly
    pos1 = CS.local_positions(40, 1, 2)
    assert pos1.numel() == 0
    a = CS.partial_attention(q[:1], k[:40], v[:40], torch.arange(40), torch.tensor([39]), 0.1)
    b = CS.partial_attention(q[:1], k[:0], v[:0], pos1, torch.tensor([39]), 0.1)
    assert torch.allclose(CS.merge_partials([a, b]), R.causal_attention(q[:1], k[:40], v[:40], 39, 0.1).float(), atol=1e-5)


def test_candidate_merge_is_the_global_topk():
    g = torch.Generator().manual_seed(1)
    Tk, R_, k = 500, 4, 16
    s = torch.randn(R_, Tk, generator=g)
    s[:, 10] = s[:, 200]                                      # a tie across ranks
    sc, ps = [], []
    for r in range(2):
        pos = CS.local_positions(Tk, r, 2)
        loc = s[:, pos]
        top = torch.sort(loc, dim=1, descending=True, stable=True).indices[:, :k]
        sc.append(loc.gather(1, top)); ps.append(pos[top])
    got = CS.merge_candidates(sc, ps, k)
    for r in range(R_):
        order = sorted(range(Tk), key=lambda i: (-float(s[r, i]), i))[:k]
        assert got[r].tolist() == sorted(order)


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(3)                      # same tensors on every rank
    Tk, Tq, H, Hk, D = 260, 4, 8, 2, 32
    q, k, v = torch.randn(Tq, H, D, generator=g), torch.randn(Tk, Hk, D, generator=g), torch.randn(Tk, Hk, D, generator=g)
    cs = CS.ContextSplit()
    hn = H // world
    pos = CS.local_positions(Tk, rank, world)
    own = cs.attend(q[:, rank * hn:(rank + 1) * hn], k[pos], v[pos], pos, torch.arange(Tk - Tq, Tk))
    want = R.causal_attention(q, k, v, Tk - Tq).float()[:, rank * hn:(rank + 1) * hn]
    err = (own - want).abs().max().item()
    sel = cs.exchange_candidates(torch.full((Tq, 3), float(rank)), torch.arange(3).repeat(Tq, 1) + 10 * rank, 4)
    torch.save({"err": err, "sel": sel}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_context_split_over_two_ranks(tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    for r in range(2):
        d = torch.load(str(tmp_path / f"r{r}.pt"))
        assert d["err"] < 1e-5
        assert d["sel"][0].tolist() == [0, 10, 11, 12]          # rank 1's three candidates win, one of rank 0's ties (lowest position); ascending output


def _decoder_worker(rank, world, port, out_dir):
    import torch.distributed as dist
    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.ref.context import ContextSplitDecoder
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = tiny_moe().replace(family="qwen3_moe", attention="gqa", num_heads=4, num_kv_heads=2, head_dim=32, hidden=128, qk_norm=True,
                             rope_interleaved=False, num_shared_experts=0, scoring="softmax")
    params = init_weights(cfg, seed=0)
    toks = torch.randint(0, cfg.vocab_size, (150,), generator=torch.Generator().manual_seed(9))      # more than two pages
    whole, split = RefDecoder(cfg, params), ContextSplitDecoder(cfg, params)
    kv_w, kv_s = KvState(cfg), split.new_kv()
    with torch.no_grad():
        errs = [(split.forward(toks[:140], kv_s) - whole.forward(toks[:140], kv_w)).abs().max().item()]
        for t in range(140, 150):                              # decode steps: each row lands on the owner of its page
            errs.append((split.forward(toks[t:t + 1], kv_s) - whole.forward(toks[t:t + 1], kv_w)).abs().max().item())
    torch.save({"err": max(errs), "held": kv_s.held(0), "total": kv_s.length(0)}, os.path.join(out_dir, f"d{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_whole_decoder_with_context_split_attention(tmp_path):
    """Prompt + decode through a full model whose attention runs context-split over two ranks: same logits, and every
    rank keeps only the KV rows of its pages."""
    import torch.multiprocessing as mp
    mp.spawn(_decoder_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    d0, d1 = (torch.load(str(tmp_path / f"d{r}.pt")) for r in range(2))
    assert d0["err"] < 2e-3 and d1["err"] < 2e-3                 # fp32 oracle: only the summation order differs
    assert d0["total"] == d1["total"] == 150
    assert d0["held"] == 64 + 22 and d1["held"] == 64            # pages 0 and 2 (positions 0..63, 128..149) / page 1
