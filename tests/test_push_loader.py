"""Push loader over gloo CPU ranks: the coordinator reads every owned tensor once and each rank ends up with exactly
the pieces the owners function names (whole tensors, row windows, replicated tensors, E4M3 payloads)."""
import os
import socket

import torch

from cuteafd_b200.loader.safetensors_io import write_sharded


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _tensors():
    g = torch.Generator().manual_seed(0)
    t = {"model.embed_tokens.weight": torch.randn(64, 16, generator=g).to(torch.bfloat16),
         "model.norm.weight": torch.ones(16, dtype=torch.bfloat16),
         "unused.bias": torch.randn(7, generator=g)}
    for e in range(6):
        t[f"model.layers.0.mlp.experts.{e}.up_proj.weight"] = torch.randn(8, 128, generator=g).to(torch.float8_e4m3fn)
        t[f"model.layers.0.mlp.experts.{e}.up_proj.weight_scale_inv"] = torch.rand(1, 1, generator=g)
    t["lm_head.weight"] = torch.randn(96, 16, generator=g).to(torch.bfloat16)
    return t


def _owners(name, shape):
    from cuteafd_b200.loader.push import expert_parallel_owners
    if name == "unused.bias":
        return []
    if name == "lm_head.weight":                        # vocabulary-sharded head over the two attention ranks
        return [(0, 0, 48), (1, 48, -1)]
    return expert_parallel_owners([0, 1], [2, 3], 6)(name, shape)


def _worker(rank, world, port, directory, out_dir):
    import torch.distributed as dist

    from cuteafd_b200.loader.push import push_load
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    seen = []
    mine, stats = push_load(directory if rank == 0 else None, _owners if rank == 0 else None, ring=2,
                            transform=lambda name, first, t: (seen.append(name), t)[1])
    torch.save({"mine": mine, "stats": stats.__dict__, "seen": seen}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_push_load_delivers_owned_pieces(tmp_path):
    import torch.multiprocessing as mp
    src = str(tmp_path / "snap")
    os.makedirs(src)
    ref = _tensors()
    write_sharded(src, ref, shard_bytes=4096)            # several shard files
    out = str(tmp_path / "out")
    os.makedirs(out)
    mp.spawn(_worker, args=(4, _free_port(), src, out), nprocs=4, join=True)
    got = [torch.load(os.path.join(out, f"r{r}.pt"), weights_only=False) for r in range(4)]
    same = lambda a, b: a.dtype == b.dtype and torch.equal(a.view(torch.uint8), b.contiguous().view(torch.uint8))   # noqa: E731
    for r in (0, 1):                                     # attention ranks: everything but experts, own half of the head
        m = got[r]["mine"]
        assert same(m["model.embed_tokens.weight"][0][1], ref["model.embed_tokens.weight"])
        first, piece = m["lm_head.weight"][0]
        assert first == 48 * r and same(piece, ref["lm_head.weight"][48 * r:48 * r + 48])
        assert not any(".experts." in k for k in m) and "unused.bias" not in m
    for r, ids in ((2, (0, 1, 2)), (3, (3, 4, 5))):      # expert ranks: their id range, payload and scales
        m = got[r]["mine"]
        assert sorted(m) == sorted(f"model.layers.0.mlp.experts.{e}.up_proj.{s}" for e in ids for s in ("weight", "weight_scale_inv"))
        for k, pieces in m.items():
            assert same(pieces[0][1], ref[k])
        assert len(got[r]["seen"]) == 6                  # the transform saw every landed piece
    st = got[0]["stats"]
    owned = {k: v for k, v in ref.items() if k != "unused.bias"}
    assert st["tensors_read"] == len(owned)
    assert st["bytes_read"] == sum(v.numel() * v.element_size() for v in owned.values())     # each byte read once
    assert st["bytes_sent"] > 0 and st["bytes_kept"] > 0
