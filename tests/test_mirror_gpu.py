"""A tensor-parallel attention group under one driver: rank 0 runs the generator over a mirrored engine, rank 1 repeats
its steps (parallel/mirror.py).  Logits against the fp32 oracle, eager and with rank 0 replaying CUDA graphs, and a
KV page copy that has to happen on both ranks."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, out_dir: str, family: str) -> None:
    import torch.distributed as dist

    from cuteafd_b200.ops import kernels as K
    from cuteafd_b200.parallel.mirror import FollowerStats, MirroredEngine, follow
    from cuteafd_b200.ref.model import KvState, RefDecoder, init_weights
    from cuteafd_b200.runtime.generate import Generator
    from cuteafd_b200.runtime.paged import PagePool
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    K.set_wait_limit_ns(2_000_000_000)
    if family == "mla":
        from cuteafd_b200.models.mla_moe import MlaMoeWeights as Weights
        from cuteafd_b200.models.tp_mla import TpMlaMoeEngine as Engine
        from tests.test_mla_gpu import _mla_cfg
        cfg = _mla_cfg()
    else:
        from cuteafd_b200.models.gqa_moe import GqaMoeWeights as Weights
        from cuteafd_b200.models.tp_gqa import TpGqaMoeEngine as Engine
        from tests.test_tp_engine_gpu import _cfg
        cfg = _cfg()
    params = {k: v.to(torch.bfloat16).float() for k, v in init_weights(cfg, seed=0).items()}
    inner = Engine(cfg, Weights.from_params(cfg, params, dev), num_pages=64, max_tokens=256, max_seqs=8)
    pool_of = (lambda kv: kv.c[0]) if family == "mla" else (lambda kv: kv.k[0])
    dist.barrier()
    if rank != 0:
        st = FollowerStats()
        steps = follow(inner, stats=st)
        torch.cuda.synchronize()
        page = pool_of(inner.kv)
        torch.save({"steps": steps, "status": K.read_status(), "captures": st.captures, "replays": st.replays, "copied": bool(torch.equal(page[1], page[60])) and bool(page[1].abs().sum() > 0)},
                   os.path.join(out_dir, f"r{rank}.pt"))
        dist.barrier()
        dist.destroy_process_group()
        return
    eng = MirroredEngine(inner)
    ref = RefDecoder(cfg, params)
    errs = {}
    for use_graphs in (False, True):
        gen = Generator(eng, PagePool(56), max_pages_per_seq=8, max_seqs=8, prefill_chunk=128, use_graphs=use_graphs)
        g = torch.Generator().manual_seed(1)
        prompts = [torch.randint(0, cfg.vocab_size, (n,), generator=g) for n in (200, 77, 5)]
        seqs, last, kvs_all, e = [], [], [], []
        with torch.no_grad():
            for p in prompts:
                s = gen.table.new()
                gen.prefill(s, p.tolist())
                kvs = KvState(cfg)
                rl = ref.forward(p, kvs)[-1]
                e.append((eng.logits[0].float().cpu() - rl).abs().max().item() / max(rl.abs().max().item(), 1.0))
                seqs.append(s); kvs_all.append(kvs); last.append(int(rl.argmax()))
            for step in range(4):
                gen.decode(seqs, last)
                torch.cuda.synchronize()
                assert K.read_status() == 0
                for i in range(len(seqs)):
                    rl = ref.forward(torch.tensor([last[i]]), kvs_all[i])[-1]
                    e.append((eng.logits[i].float().cpu() - rl).abs().max().item() / max(rl.abs().max().item(), 1.0))
                    last[i] = int(rl.argmax())
        errs["graphs" if use_graphs else "eager"] = e
    eng.kv.copy_page(1, 60)                      # copy-on-write of a shared page: every rank copies its own heads' page
    eng.stop()
    torch.cuda.synchronize()
    page = pool_of(inner.kv)
    torch.save({"errs": errs, "status": K.read_status(), "mirrored": eng.mirrored_steps, "copied": bool(torch.equal(page[1], page[60]))},
               os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("family", ["gqa", "mla"])
def test_followers_repeat_rank_zero(family, tmp_path):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs 2 GPUs")
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path), family), nprocs=2, join=True)
    lead, fol = torch.load(str(tmp_path / "r0.pt")), torch.load(str(tmp_path / "r1.pt"))
    assert lead["status"] == 0 and fol["status"] == 0
    for mode, e in lead["errs"].items():
        e = sorted(e)
        assert e[len(e) // 2] < 0.03 and e[-1] < 0.25, (mode, e)
    assert fol["steps"] == lead["mirrored"] > 0 and lead["copied"] and fol["copied"]
    assert fol["captures"] >= 1 and fol["replays"] >= 4           # the follower's own graph of the 3-sequence decode step
