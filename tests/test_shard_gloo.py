"""Multi-process (world_size 2 and 3, gloo, CPU) tests of the partitioning used for N > 1 GPUs: batch slices,
(batch, head group) slabs of the dense operator, square blocks of one item's scores with the two all-reduces of the
d_q / d_k partial sums, and the sparse operator by dst-token range with its one
all-reduce of the d_k / d_v partial sums.  The compute itself is a pure-torch stand-in here (the library has no
CPU path); what is tested is the partition, the placement of the pieces and the collectives."""
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


# ------------------------------------------------------------------ (batch, head group) slabs

def test_dense_partition_covers_every_batch_head_pair_once():
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    for bs, heads, world in [(16, 16, 8), (2, 8, 8), (2, 8, 4), (2, 8, 2), (3, 5, 7), (1, 16, 3), (5, 4, 2)]:
        part = sh.dense_partition(bs, heads, world)
        assert len(part) == world
        seen = torch.zeros(bs, heads, dtype=torch.int32)
        for b0, b1, h0, h1 in part:
            assert b1 > b0 and h1 > h0
            seen[b0:b1, h0:h1] += 1
        assert bool((seen == 1).all()), (bs, heads, world)
    assert sh.dense_partition(2, 8, 8)[5] == (1, 2, 2, 4)        # long-context shape on 8 ranks: 2 heads each
    assert sh.dense_partition(16, 16, 8)[3] == (6, 8, 0, 16)     # benchmark shape: 2 batch items, all heads
    with pytest.raises(ValueError):
        sh.dense_partition(1, 2, 3)


def _torch_scores(q, k):
    return -(q[:, None, :, :, :] - k[:, :, None, :, :]).abs().sum(-1) / q.shape[-1] ** 0.5  # [b, s, t, h]


def _dense_worker(rank, world, port, shape, q):
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bs, n, h, w = shape
        g = torch.Generator().manual_seed(3)
        qq, kk = torch.randn(shape, generator=g), torch.randn(shape, generator=g)
        slab = sh.dense_partition(bs, h, world)[rank]
        local = _torch_scores(sh.dense_local(qq, slab), sh.dense_local(kk, slab))
        full = sh.gather_dense(local, bs, h)
        q.put((rank, bool(torch.equal(full, _torch_scores(qq, kk)))))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape", [(2, (4, 6, 4, 5)), (3, (2, 5, 6, 4)), (2, (1, 7, 3, 2))])
def test_head_group_shards_assemble_to_the_global_scores(world, shape):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() * 11 + world * 17 + shape[0]) % 2000
    procs = [ctx.Process(target=_dense_worker, args=(r, world, port, shape, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok in res)


# ------------------------------------------------------------------ square blocks of one item's scores

def test_grid_partition_tiles_every_score_once_and_names_the_right_partners():
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    for bs, heads, n, world in [(2, 8, 4096, 8), (1, 16, 64, 8), (1, 8, 32, 8), (1, 4, 6, 4), (2, 8, 16, 4), (3, 5, 10, 7),
                                (16, 16, 8, 8), (1, 32, 12, 16), (1, 8, 7, 4)]:
        part = sh.dense_grid_partition(bs, heads, n, world)
        assert len(part) == world
        seen = torch.zeros(bs, n, n, heads, dtype=torch.int32)
        for r, p in enumerate(part):
            assert p["t1"] - p["t0"] == p["s1"] - p["s0"], "blocks must be square problems"
            seen[p["b0"]:p["b1"], p["s0"]:p["s1"], p["t0"]:p["t1"], p["h0"]:p["h1"]] += 1
            assert r in p["row"] and r in p["col"]
            same = lambda a, b, keys: all(a[x] == b[x] for x in keys)
            for o, po in enumerate(part):  # partners: exactly the ranks with the same (b, heads, query / key block)
                assert (o in p["row"]) == same(p, po, ("b0", "b1", "h0", "h1", "t0", "t1"))
                assert (o in p["col"]) == same(p, po, ("b0", "b1", "h0", "h1", "s0", "s1"))
        assert bool((seen == 1).all()), (bs, heads, n, world)
    cfg3 = sh.dense_grid_partition(2, 8, 4096, 8)  # long-context shape on 8 ranks: all heads, 2 x 2 blocks per item
    assert [cfg3[5][x] for x in ("b0", "h0", "h1", "t0", "t1", "s0", "s1")] == [1, 0, 8, 0, 2048, 2048, 4096]
    assert cfg3[5]["row"] == [4, 5] and cfg3[5]["col"] == [5, 7]
    odd = sh.dense_grid_partition(1, 8, 7, 4)      # 7 tokens cannot be halved: plain head groups
    assert all(p["t1"] - p["t0"] == 7 and p["h1"] - p["h0"] == 2 for p in odd)
    with pytest.raises(ValueError):
        sh.dense_grid_partition(1, 2, 9, 3)


class _TorchDenseOps:
    """Stand-in for the single-GPU dense operator on the CPU (differentiable torch)."""

    def forward(self, q, k, out):
        return _torch_scores(q, k)

    def backward(self, d_attn, q, k, out, scratch):
        q, k = q.detach().clone().requires_grad_(True), k.detach().clone().requires_grad_(True)
        _torch_scores(q, k).backward(d_attn)
        return q.grad, k.grad

    def scratch(self, q):
        return None


def _grid_worker(rank, world, port, shape, q):
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        bs, n, h, w = shape
        g = torch.Generator().manual_seed(7)
        qq, kk = (torch.randn(shape, generator=g, dtype=torch.float64) for _ in range(2))
        d_attn = torch.randn(bs, n, n, h, generator=g, dtype=torch.float64)
        ops = _TorchDenseOps()
        plan = sh.DenseGridShard(bs, n, h, rank, world, ops=ops)
        ql, kl = plan.local_inputs(qq, kk)
        attn = plan.forward(ql, kl)
        dq, dk = plan.backward(plan.local_scores(d_attn), ql, kl)
        ref = _torch_scores(qq, kk)
        rdq, rdk = ops.backward(d_attn, qq, kk, None, None)
        m = plan.me
        close = lambda a, b: bool(torch.allclose(a, b, rtol=1e-12, atol=1e-12))
        ok = (close(attn, plan.local_scores(ref))
              and close(dq, rdq[m["b0"]:m["b1"], m["t0"]:m["t1"], m["h0"]:m["h1"]])
              and close(dk, rdk[m["b0"]:m["b1"], m["s0"]:m["s1"], m["h0"]:m["h1"]]))
        q.put((rank, ok, plan.collective_note() is not None, plan.describe()))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,shape,exchange", [(4, (1, 6, 4, 3), True), (2, (1, 6, 4, 3), False), (3, (4, 5, 2, 3), False)])
def test_square_block_shards_give_the_global_gradients(world, shape, exchange):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 35500 + (os.getpid() * 17 + world * 23 + shape[0]) % 2000
    procs = [ctx.Process(target=_grid_worker, args=(r, world, port, shape, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, ok, _, _ in res), res
    assert all(ex == exchange for _, _, ex, _ in res), res


# ------------------------------------------------------------------ sparse by dst-token range

class _TorchSparseOps:
    """Stand-in compute backend for SparseShard on the CPU: the operator's math in differentiable torch
    (scatter form), the edge index replaced by the expanded list itself."""

    def expand(self, co):
        from oracle import oracle
        coo, dm, _ = oracle.expand_coo(co.numpy())
        return torch.from_numpy(coo), dm

    def index(self, coo, n_tok, dst_mxlen):
        return coo.long()

    @staticmethod
    def _vo(v, q, k, coo, usm):
        dst, src = coo[:, 0], coo[:, 1]
        x = -(q[:, dst] - k[:, src]).abs().sum(-1) / q.shape[-1] ** 0.5
        e = torch.exp(x)
        a = e / torch.ones_like(q[..., 0]).index_add(1, dst, e)[:, dst] if usm else e
        return torch.zeros_like(v).index_add(1, dst, a.unsqueeze(-1) * v[:, src]), a

    def forward(self, v, q, k, ix, usm, out):
        vo, a = self._vo(v, q, k, ix, usm)
        out[0].copy_(vo)
        out[1].zero_()
        out[1][:, ix[:, 0], ix[:, 2]] = a
        return out

    def backward(self, dvo, v, q, k, ix, attn, usm, out, scratch):
        v, q, k = (t.detach().clone().requires_grad_(True) for t in (v, q, k))
        self._vo(v, q, k, ix, usm)[0].backward(dvo)
        for o, t in zip((out[0], out[2], out[3]), (v, q, k)):
            o.copy_(t.grad if t.grad is not None else torch.zeros_like(t))


def _sparse_worker(rank, world, port, bs, mode, q):
    sys.path.insert(0, PKG)
    import l1attn_shard as sh
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        n, h, w = 11, 2, 4
        g = torch.Generator().manual_seed(5)
        co = torch.stack([torch.randint(0, n, (60,), generator=g), torch.randint(0, n, (60,), generator=g)], 1)
        v, qq, kk, dvo = (torch.randn(bs, n, h, w, generator=g, dtype=torch.float64) for _ in range(4))
        ops = _TorchSparseOps()
        plan = sh.SparseShard(co, bs, n, rank, world, device="cpu", ops=ops, n_heads=h, mode=mode)
        vo, dv, dq, dk = plan.forward_backward(v, qq, kk, dvo, True)
        whole = sh.SparseShard(co, bs, n, 0, 1, device="cpu", ops=ops)
        rvo, rdv, rdq, rdk = whole.forward_backward(v, qq, kk, dvo, True)
        close = lambda a, b: bool(torch.allclose(a, b, rtol=1e-12, atol=1e-12))
        if plan.mode in ("batch", "head"):
            sl = (slice(plan.b0, plan.b1), slice(None), slice(plan.h0, plan.h1))
            ok = close(vo, rvo[sl]) and close(dv, rdv[sl]) and close(dq, rdq[sl]) and close(dk, rdk[sl])
            ok = ok and plan.collective_note() is None
        else:
            rows = slice(plan.d0, plan.d1)
            outside = torch.ones(n, dtype=torch.bool)
            outside[rows] = False
            ok = (close(vo[:, rows], rvo[:, rows]) and close(dq[:, rows], rdq[:, rows])   # owned dst rows complete
                  and float(vo[:, outside].abs().sum()) == 0 and float(dq[:, outside].abs().sum()) == 0
                  and close(dv, rdv) and close(dk, rdk))                                  # summed over the ranks
            ok = ok and plan.collective_note() is not None
        q.put((rank, plan.mode, ok, plan.n_edges_local))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,bs,mode,want", [(2, 1, "dst", "dst"), (3, 2, "dst", "dst"), (2, 4, "auto", "batch"),
                                                (2, 1, "auto", "head"), (3, 2, "auto", "head")])
def test_sparse_dst_range_head_and_batch_shards(world, bs, mode, want):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 33500 + (os.getpid() * 13 + world * 19 + bs + 7 * len(mode)) % 2000
    procs = [ctx.Process(target=_sparse_worker, args=(r, world, port, bs, mode, q)) for r in range(world)]
    for p in procs:
        p.start()
    res = sorted(q.get(timeout=120) for _ in range(world))
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert all(ok for _, _, ok, _ in res), res
    assert {m for _, m, _, _ in res} == {want}
    if want == "dst":
        assert sum(e for _, _, _, e in res) == 60  # every edge on exactly one rank
