"""Failure detection on the host: a rank that leaves between steps is noticed by the others before their next launch
(no GPU involved: two gloo ranks on the CPU, the failure is made by the test itself)."""
import os
import time

import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from polarengine_vllm_b200.health import PeerLeft, PeerStale, RankMonitor


def _worker(rank, world, port, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    store = dist.distributed_c10d._get_default_store()
    mon = RankMonitor(store, rank, world, prefix="t1")
    try:
        t = torch.ones(4)
        for step in range(1, 6):
            if rank == 1 and step == 3:
                mon.leave("injected: rank 1 stops after step 2")   # between steps, nothing in flight
                return
            if rank == 0 and step == 3:
                deadline = time.time() + 20.0
                while time.time() < deadline:       # rank 1's note arrives through the store, not through a collective
                    try:
                        mon.check()
                    except PeerLeft as e:
                        ret["left"] = (e.rank, e.reason, step)
                        return
                    time.sleep(0.05)
                ret["left"] = None
                return
            mon.check()
            dist.all_reduce(t)                       # the step's exchange
            mon.beat(step)
        ret["finished"] = True
    finally:
        if rank == 0:
            ret["sum"] = float(t[0])
        # no destroy_process_group: the survivor must not wait for the rank that left


def test_rank_that_leaves_between_steps_is_noticed_before_the_next_launch():
    ctx = mp.get_context("spawn")
    ret = ctx.Manager().dict()
    port = 29650 + os.getpid() % 200
    procs = [ctx.Process(target=_worker, args=(r, 2, port, ret)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(90)
        assert not p.is_alive()
    assert ret.get("left") == (1, "injected: rank 1 stops after step 2", 3)
    assert ret.get("sum") == 4.0 and "finished" not in ret     # two completed steps (1 -> 2 -> 4), none attempted after


class _DictStore:
    """The three store calls the monitor uses, in memory."""

    def __init__(self):
        self.d = {}

    def set(self, k, v):
        self.d[k] = v.encode() if isinstance(v, str) else v

    def get(self, k):
        return self.d[k]

    def check(self, keys):
        return all(k in self.d for k in keys)


def test_stale_peer_is_reported():
    store = _DictStore()
    a = RankMonitor(store, 0, 2, stale_after_s=0.05)
    b = RankMonitor(store, 1, 2)
    b.beat(7)
    a.check()                       # first sight of counter 7
    time.sleep(0.1)
    try:
        a.check()
        raise AssertionError("a peer whose counter stands still must be reported")
    except PeerStale as e:
        assert e.rank == 1 and e.age_s >= 0.05
    b.beat(8)
    a.check()                       # moving again
    b.leave("done")
    try:
        a.check()
        raise AssertionError("a farewell note must be reported")
    except PeerLeft as e:
        assert (e.rank, e.reason) == (1, "done")
