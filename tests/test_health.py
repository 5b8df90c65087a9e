"""Failure detection on the host: latch semantics, heartbeat over a store with gloo CPU ranks, a rank that leaves
between steps, a rank that dies silently.  No GPU involved."""
import os
import socket
import time

import pytest
import torch.multiprocessing as mp

from cuteafd_b200.parallel.health import Heartbeat, HealthError, HealthLatch, PeerState


class DictStore:
    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v

    def get(self, k):
        return self.d[k].encode()

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_latch_is_terminal_and_keeps_first_reason():
    L = HealthLatch()
    L.require()
    assert L.trip("peer 3 timed out") and not L.trip("later noise")
    assert L.reason == "peer 3 timed out" and L.state is PeerState.ABORTING
    with pytest.raises(HealthError, match="peer 3"):
        L.require()
    L.drained(success=False)
    assert L.state is PeerState.RETAINED
    L2 = HealthLatch()
    L2.check_device(0)
    assert L2.ok
    L2.check_device(5, "fc1")
    assert "peer flag" in L2.reason and "fc1" in L2.reason


def test_heartbeat_detects_silence_and_orderly_exit():
    store, latch = DictStore(), HealthLatch()
    me = Heartbeat(store, 0, 3, latch, timeout=1.0)
    store.set("hb/1", "7"); store.set("hb/2", "4")
    me.check(now=100.0)
    store.set("hb/1", "8")                      # rank 1 keeps beating, rank 2 is silent
    me.check(now=100.9)
    assert latch.ok
    me.check(now=101.2)
    assert not latch.ok and "rank 2" in latch.reason
    latch2 = HealthLatch()
    me2 = Heartbeat(store, 0, 3, latch2, timeout=1.0)
    store.set("leaving/1", "1")
    me2.check(now=5.0)
    assert "rank 1 left" in latch2.reason


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _rank(rank, world, port, out_dir, mode):
    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    latch = HealthLatch()
    hb = Heartbeat(store, rank, world, latch, period=0.05, timeout=0.6).start()
    steps = 0
    t = torch.ones(1)
    for step in range(200):
        hb.check()
        if not latch.ok:
            break                                   # refuse to launch the next step
        if rank == world - 1 and step == 3:
            if mode == "leave":
                hb.leave()                          # orderly: between steps, nothing in flight
            else:
                hb.stop()                           # silent death of the beating thread
            break
        dist.all_reduce(t) if step < 3 else time.sleep(0.05)     # collectives only while everyone is known alive
        steps += 1
    with open(os.path.join(out_dir, f"r{rank}.txt"), "w") as f:
        f.write(f"{steps}|{latch.reason}")
    time.sleep(1.0 if rank == 0 else 0.2)           # rank 0 hosts the store: let the others finish reading it
    os._exit(0)


@pytest.mark.parametrize("mode", ["leave", "silent"])
def test_ranks_learn_of_a_lost_peer_between_steps(tmp_path, mode):
    world = 3
    mp.spawn(_rank, args=(world, _free_port(), str(tmp_path), mode), nprocs=world, join=True)
    for r in range(world - 1):
        steps, reason = open(tmp_path / f"r{r}.txt").read().split("|")
        assert int(steps) >= 3 and f"rank {world - 1}" in reason, (r, steps, reason)
