"""Multi-process (world_size 2 and 3, gloo, CPU) tests of the batch partitioning used for N > 1 GPUs."""
import os
import sys

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from conftest import PKG


def _worker(rank, world, port, n_total, q):
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        lo, hi = sh.shard_range(n_total, rank, world)
        full = torch.arange(n_total * 6, dtype=torch.float32).reshape(n_total, 2, 3)
        got = sh.gather_batch(full[lo:hi].clone(), n_total)
        slow = sh.max_over_ranks(10.0 + rank)
        q.put((rank, lo, hi, bool(torch.equal(got, full)), slow))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n_total", [(2, 16), (2, 5), (3, 2)])
def test_partition_gather_and_max(world, n_total):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() * 7 + world * 13 + n_total) % 2000
    procs = [ctx.Process(target=_worker, args=(r, world, port, n_total, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    covered = []
    for rank, lo, hi, same, slow in res:
        covered += list(range(lo, hi))
        assert same, "gathered tensor differs on rank %d" % rank
        assert slow == 10.0 + world - 1
    assert covered == list(range(n_total))  # disjoint, ordered, complete
    sizes = [hi - lo for _, lo, hi, _, _ in res]
    assert max(sizes) - min(sizes) <= 1


def test_shard_range_errors_and_single_process():
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    assert sh.shard_range(16, 0, 1) == (0, 16)
    assert [sh.shard_range(10, r, 4) for r in range(4)] == [(0, 3), (3, 6), (6, 8), (8, 10)]
    with pytest.raises(ValueError):
        sh.shard_range(4, 4, 4)
    assert sh.max_over_ranks(3.5) == 3.5
    t = torch.ones(2, 3)
    assert sh.gather_batch(t, 2) is t
