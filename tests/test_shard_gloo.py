"""world_size-2 (and 3) CPU tests of the multi-GPU host logic over the gloo backend:
shard bounds, ragged all-gather in rank order, max-over-ranks timing, and a rank that raises
before the collective (the others learn of it on the host within a time limit and keep their own
shard instead of hanging in the all-gather)."""
import datetime
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from cssm_b200 import shard


def test_shard_bounds_cover_and_balance():
    for n in (0, 1, 7, 128, 129):
        for world in (1, 2, 3, 8):
            b = [shard.shard_bounds(n, r, world) for r in range(world)]
            assert b[0][0] == 0 and b[-1][1] == n
            assert all(b[i][1] == b[i + 1][0] for i in range(world - 1))
            sizes = [hi - lo for lo, hi in b]
            assert max(sizes) - min(sizes) <= 1
            assert sizes == shard.shard_sizes(n, world)
    with pytest.raises(ValueError):
        shard.shard_bounds(4, 2, 2)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, n, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(n * 3, dtype=torch.float32).reshape(n, 3)
        lo, hi = shard.shard_bounds(n, rank, world)
        local = full[lo:hi] * 2.0 + 1.0            # stand-in for the per-sample forward
        got = shard.gather_outputs(local, n)
        slow = shard.max_over_ranks(10.0 + rank, "cpu")
        ok = torch.equal(got, full * 2.0 + 1.0) and slow == 10.0 + world - 1
        try:
            shard.gather_outputs(local[:-1] if local.shape[0] else torch.zeros(1, 3), n)
            ok = False                              # wrong shard size must raise
        except ValueError:
            pass
        q.put((rank, bool(ok)))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n", [(2, 8), (2, 7), (3, 10)])
def test_gather_rank_order_over_gloo(world, n):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, n, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = dict(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert res == {r: True for r in range(world)}


def _failing_worker(rank, world, port, store_port, n, q):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    store = dist.TCPStore("127.0.0.1", store_port, world, is_master=(rank == 0),
                          timeout=datetime.timedelta(seconds=60))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        full = torch.arange(n * 2, dtype=torch.float32).reshape(n, 2)
        lo, hi = shard.shard_bounds(n, rank, world)
        local = full[lo:hi] + 0.5
        # step 0: everybody is there
        got, err = shard.gather_outputs_checked(local, n, store, step=0, timeout_s=30.0)
        ok0 = err is None and torch.equal(got, full + 0.5)
        # step 1: the last rank fails before the collective (between steps, nothing in flight)
        if rank == world - 1:
            q.put((rank, ok0, "raised"))
            raise RuntimeError("injected failure before the collective")
        got, err = shard.gather_outputs_checked(local, n, store, step=1, timeout_s=2.0)
        ok1 = isinstance(err, shard.PeerTimeout) and err.missing == [world - 1] and torch.equal(got, local)
        q.put((rank, ok0 and ok1, "reported"))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world", [2, 3])
def test_rank_that_raises_before_the_gather_is_reported(world):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port, store_port = _free_port(), _free_port()
    procs = [ctx.Process(target=_failing_worker, args=(r, world, port, store_port, 9, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = {}
    for _ in range(world):
        r, ok, what = q.get(timeout=120)
        res[r] = (ok, what)
    for p in procs:
        p.join(timeout=60)
    assert res[world - 1] == (True, "raised") and procs[world - 1].exitcode != 0
    for r in range(world - 1):
        assert res[r] == (True, "reported") and procs[r].exitcode == 0
