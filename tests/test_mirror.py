"""The mirror protocol over gloo CPU ranks with a recording stand-in for the engine: every forward step and KV page
copy of rank 0 arrives on the follower with the same contents, in order, until the stop message."""
import os
import socket

import torch


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


class _Kv:
    def __init__(self):
        self.copies = []

    def copy_page(self, src, dst):
        self.copies.append((src, dst))


class _Engine:
    """Records what it is asked to run."""
    device = torch.device("cpu")

    def __init__(self):
        self.kv, self.seen = _Kv(), []

    def forward(self, b):
        self.seen.append({"tokens": b.tokens.tolist(), "positions": b.positions.tolist(), "slots": b.slots.tolist(),
                          "table": b.page_table.tolist(), "lens": b.seq_lens.tolist(), "q_start": b.q_start.tolist(),
                          "max_q_len": b.max_q_len, "prefill": b.prefill, "fresh": b.fresh,
                          "last": None if b.last_rows is None else b.last_rows.tolist()})
        return torch.zeros(1)

    def mtp_forward(self, *a):
        raise AssertionError("not mirrored")


def _batches():
    from cuteafd_b200.models.gqa_moe import Batch
    i32 = lambda v: torch.tensor(v, dtype=torch.int32)                      # noqa: E731
    return [Batch(i32([5, 6, 7]), i32([0, 1, 2]), i32([64, 65, 66]), i32([[1, 0, 0]]), i32([3]), i32([0, 3]), 3, True, i32([2]), fresh=True),
            Batch(i32([9, 4]), i32([3, 17]), i32([67, 145]), i32([[1, 0, 0], [2, 3, 0]]), i32([4, 18]), i32([0, 1, 2]), 1, False, None)]


def _worker(rank: int, world: int, port: int, out_dir: str) -> None:
    import torch.distributed as dist

    from cuteafd_b200.parallel.mirror import MirroredEngine, follow
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    inner = _Engine()
    if rank == 0:
        eng = MirroredEngine(inner)
        assert not hasattr(eng, "mtp_forward") and eng.device.type == "cpu"      # the MTP depth is hidden, the rest passes through
        bs = _batches()
        eng.forward(bs[0])
        eng.kv.copy_page(3, 9)
        eng.forward(bs[1])
        eng.mirror(bs[1])                                # what the graph bank does before a replay
        eng.stop()
        steps = eng.mirrored_steps
    else:
        steps = follow(inner)
    torch.save({"seen": inner.seen, "copies": inner.kv.copies, "steps": steps}, os.path.join(out_dir, f"r{rank}.pt"))
    dist.barrier()
    dist.destroy_process_group()


def test_follower_sees_every_step_and_copy(tmp_path):
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(2, _free_port(), str(tmp_path)), nprocs=2, join=True)
    lead, fol = torch.load(str(tmp_path / "r0.pt")), torch.load(str(tmp_path / "r1.pt"))
    assert lead["steps"] == fol["steps"] == 3 and fol["copies"] == lead["copies"] == [(3, 9)]
    assert fol["seen"][:2] == lead["seen"] and fol["seen"][2] == lead["seen"][1]
    assert fol["seen"][0]["fresh"] and fol["seen"][0]["last"] == [2] and fol["seen"][1]["last"] is None
