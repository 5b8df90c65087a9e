"""Pipeline hop and vocabulary-sharded head over gloo CPU ranks."""
import os
import socket

import torch
import torch.multiprocessing as mp


def _port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, out_dir):
    import torch.distributed as dist

    from cuteafd_b200.parallel.head import ShardedHead, shard_rows
    from cuteafd_b200.parallel.pp import Hop, StagePlan, run_pipelined
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    g = torch.Generator().manual_seed(0)
    # ---- pipeline: 6 layers of y = tanh(x W_l) over 2 stages, 3 micro-batches -------------------------------
    Ws = [torch.randn(32, 32, generator=g) * 0.3 for _ in range(6)]
    mbs = [torch.randn(5, 32, generator=g) for _ in range(3)]
    plan = StagePlan.even(6, world)
    assert [plan.stage_of(l) for l in range(6)] == [0, 0, 0, 1, 1, 1]

    def stage_fn(x):
        for l in plan.layers(rank):
            x = torch.tanh(x @ Ws[l])
        return x
    prev = Hop(rank - 1) if rank > 0 else None
    nxt = Hop(rank + 1) if rank < world - 1 else None
    outs = run_pipelined(rank, world, mbs, stage_fn, prev, nxt, torch.empty_like)
    if rank == world - 1:
        for x, y in zip(mbs, outs):
            ref = x
            for W in Ws:
                ref = torch.tanh(ref @ W)
            assert torch.allclose(y, ref, atol=1e-6)
        assert prev.bytes_moved == 3 * 5 * 32 * 4
    # ---- sharded head: ties, a NaN, vocabulary not divisible by the tile ---------------------------------------
    V, H, T = 1000, 16, 7
    head = torch.randn(V, H, generator=g)
    x = torch.randn(T, H, generator=g)
    head[700] = head[3]                                  # exact tie between two ranks' slices: the lower id wins
    lo, hi = shard_rows(V, world, rank)
    sh = ShardedHead(head[lo:hi], V, linear=lambda a, w: a @ w.T, argmax=lambda lg: lg.argmax(1))
    full = x @ head.T
    want = torch.tensor([int(torch.nonzero(full[t] == full[t].max())[0]) for t in range(T)])
    assert torch.equal(sh.greedy(x), want)
    assert torch.allclose(sh.gather_logits(x), full, atol=1e-5)
    open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    dist.barrier()
    dist.destroy_process_group()


def test_pipeline_hop_and_sharded_head(tmp_path):
    mp.spawn(_worker, args=(2, _port(), str(tmp_path)), nprocs=2, join=True)
    assert all(os.path.exists(tmp_path / f"ok{r}") for r in range(2))


def _pp_worker(rank, world, port, out_dir):
    import torch.distributed as dist

    from cuteafd_b200 import tiny_moe
    from cuteafd_b200.parallel.pp import StagePlan
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    from cuteafd_b200.ref.pipeline import PipelinedDecoder
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    cfg = tiny_moe().replace(num_layers=4, first_dense_layers=1)
    params = init_weights(cfg, seed=2)
    plan = StagePlan.even(cfg.num_layers, world)
    pd = PipelinedDecoder(RefDecoder(cfg, params), plan, rank)
    kv = KvState(cfg)
    toks = torch.arange(3, 15) % cfg.vocab_size
    got = []
    nxt = torch.zeros(1, dtype=torch.long)
    for step in range(4):
        logits = pd.forward(toks, kv)
        if rank == world - 1:
            got.append(logits[-1].clone())
            nxt = logits[-1].argmax().view(1)
        dist.broadcast(nxt, src=world - 1)              # every stage feeds the token the last stage chose
        toks = nxt.clone()
    if rank == world - 1:
        whole, wkv = RefDecoder(cfg, params), KvState(cfg)
        t = torch.arange(3, 15) % cfg.vocab_size
        errs = []
        for step in range(4):
            ref = whole.forward(t, wkv)[-1]
            errs.append((got[step] - ref).abs().max().item())
            t = ref.argmax().view(1)
        torch.save({"errs": errs, "own": [kv.length(i) for i in range(cfg.num_layers)]}, os.path.join(out_dir, "pp.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_oracle_decoder_as_pipeline_stages(tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_pp_worker, args=(2, _port(), str(tmp_path)), nprocs=2, join=True)
    d = torch.load(str(tmp_path / "pp.pt"))
    assert max(d["errs"]) == 0.0                       # same arithmetic, only the process boundary moved
    assert d["own"] == [0, 0, 15, 15]                  # the last stage cached K/V for its own layers only
