"""Partitioning of the L1-attention operators across the GPUs of one node.

Both operators are independent per batch item and per head: no reduction crosses items, in the
forward or in the backward.  So the multi-GPU form is one process per GPU, each running the
single-GPU operators on its own slice, with no collective on the data path; a gather of the
outputs is only needed if one rank wants everything.

  shard_range(n, rank, world)        contiguous, balanced slice [lo, hi) of n items for `rank`
  max_over_ranks(x)                  all-reduce MAX of a python float (for timing: slowest rank)
  gather_batch(t, n_total)           all-gather of batch slices (dim 0) into the full tensor, any rank sizes
  dense_partition(bs, heads, world)  (batch, head group) slab of every rank for the dense operator
  dense_local(t, slab)               a rank's contiguous [b0:b1, :, h0:h1, :] copy of q or k
  gather_dense(local, bs, heads)     all-gather of the [B_loc, T, T, H_loc] score slabs into [B, T, T, H]
  dense_grid_partition(...)          (batch, head group, query block, key block) of every rank: for fewer batch
                                     items than ranks, the ranks of one item tile its T x T scores with squares
  DenseGridShard                     the dense operator on that partition: square single-GPU calls, then ONE
                                     all-reduce each of d_q (over the ranks that share the query block) and d_k
  SparseShard                        the sparse operator over the ranks: by batch item when there are at
                                     least as many items as ranks, else by dst-token range with ONE
                                     all-reduce of the d_k and d_v partial sums

The collectives go through torch.distributed (NCCL on GPUs, gloo in CPU tests).
"""
import torch
import torch.distributed as dist


def shard_range(n, rank, world):
    """Balanced contiguous partition: the first n % world ranks get one extra item."""
    if world <= 0 or not (0 <= rank < world) or n < 0:
        raise ValueError("bad partition request n=%r rank=%r world=%r" % (n, rank, world))
    base, extra = divmod(n, world)
    lo = rank * base + min(rank, extra)
    return lo, lo + base + (1 if rank < extra else 0)


def max_over_ranks(x, device=None):
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return float(x)
    t = torch.tensor([float(x)], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_batch(local, n_total):
    """All ranks receive the concatenation (dim 0) of every rank's batch slice, in rank order.
    Slices follow shard_range(n_total, rank, world) and may differ in size by one."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    sizes = [shard_range(n_total, r, world) for r in range(world)]
    lo, hi = sizes[dist.get_rank()]
    if local.shape[0] != hi - lo:
        raise ValueError("rank %d holds %d items, expected %d" % (dist.get_rank(), local.shape[0], hi - lo))
    # all_gather wants equal shapes: pad every slice to the largest one, trim after
    rows = max(h - l for l, h in sizes)
    padded = torch.zeros((rows,) + tuple(local.shape[1:]), dtype=local.dtype, device=local.device)
    padded[: hi - lo] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    return torch.cat([p[: h - l] for p, (l, h) in zip(parts, sizes)], 0)


# ------------------------------------------------------------------ dense: (batch, head group) slabs

def dense_partition(bs, n_heads, world):
    """[(b0, b1, h0, h1)] per rank.  With at least as many batch items as ranks the batch is dealt out and
    every rank keeps all heads (its q, k and score slabs are contiguous pieces of the global tensors, no
    copies).  With fewer items, the ranks are dealt out over the items and the ranks of one item split its
    heads into contiguous groups: rank-local q, k are [B_loc, T, H_loc, W] copies and the local scores
    [B_loc, T, T, H_loc] -- heads are the innermost axis of the scores, so a head shard is a strided
    interleave of the global tensor, which only gather_dense() ever materialises."""
    if bs <= 0 or n_heads <= 0 or world <= 0:
        raise ValueError("bad partition request bs=%r heads=%r world=%r" % (bs, n_heads, world))
    if bs >= world:
        return [shard_range(bs, r, world) + (0, n_heads) for r in range(world)]
    out = []
    for b in range(bs):
        r0, r1 = shard_range(world, b, bs)  # the ranks that share batch item b
        if r1 - r0 > n_heads:
            raise ValueError("%d ranks for one batch item but only %d heads" % (r1 - r0, n_heads))
        out += [(b, b + 1) + shard_range(n_heads, j, r1 - r0) for j in range(r1 - r0)]
    return out


def dense_local(t, slab):
    b0, b1, h0, h1 = slab
    return t[b0:b1, :, h0:h1].contiguous()


def gather_dense(local, bs, n_heads):
    """Every rank receives the global [bs, T, T, n_heads] scores assembled from the ranks' slabs."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size() == 1:
        return local
    world = dist.get_world_size()
    part = dense_partition(bs, n_heads, world)
    mb, mh = max(p[1] - p[0] for p in part), max(p[3] - p[2] for p in part)
    n = local.shape[1]
    padded = torch.zeros((mb, n, n, mh), dtype=local.dtype, device=local.device)
    padded[: local.shape[0], :, :, : local.shape[3]] = local
    parts = [torch.empty_like(padded) for _ in range(world)]
    dist.all_gather(parts, padded)
    full = torch.empty((bs, n, n, n_heads), dtype=local.dtype, device=local.device)
    for p, (b0, b1, h0, h1) in zip(parts, part):
        full[b0:b1, :, :, h0:h1] = p[: b1 - b0, :, :, : h1 - h0]
    return full


# ------------------------------------------------------------------ dense: square blocks of the scores of one item

def _grid_shape(n_ranks, n_heads, n_tok, lane_heads=8):
    """(head groups, g) with head groups x g x g == n_ranks: the ranks of one batch item tile its scores with
    g x g square blocks per head group; g = 1 is the plain head-group split.  Chosen for the fullest lanes: the
    forward's work item is `lane_heads` heads wide, so a rank with 2 heads runs it at a quarter of its rate;
    among equals the smallest g (least to exchange).  g must divide n_tok so that the blocks are square."""
    def fill(hs):
        h = -(-n_heads // hs)  # the widest group
        return h / float(lane_heads * -(-h // lane_heads))
    best, best_fill = (n_ranks, 1), fill(n_ranks) if n_ranks <= n_heads else -1.0
    for g in range(2, int(n_ranks ** 0.5) + 1):
        if n_ranks % (g * g) or n_tok % g:
            continue
        hs = n_ranks // (g * g)
        if hs <= n_heads and fill(hs) > best_fill + 1e-9:
            best, best_fill = (hs, g), fill(hs)
    return best


def dense_grid_partition(bs, n_heads, n_tok, world, lane_heads=8):
    """Per rank a dict(b0, b1, h0, h1, t0, t1, s0, s1, row, col): batch items, heads, query rows (t) and key rows
    (s) of its block of the scores attn[b, s, t, h]; `row` lists the ranks that hold the same (b, heads, query
    block) -- their d_q partial sums add up -- and `col` those with the same (b, heads, key block), for d_k.
    With at least as many batch items as ranks this is dense_partition(): whole items, no exchange.  Otherwise
    the ranks of one item form head groups x (g x g) square blocks, every block a square problem of n_tok / g
    tokens for the single-GPU operator.  Against splitting the heads further this keeps the head groups wide
    enough for the kernels (a rank with 2 heads runs the forward at a quarter of its rate) at the price of two
    small all-reduces in the backward."""
    if bs >= world:
        return [dict(b0=b0, b1=b1, h0=h0, h1=h1, t0=0, t1=n_tok, s0=0, s1=n_tok, row=[r], col=[r])
                for r, (b0, b1, h0, h1) in enumerate(dense_partition(bs, n_heads, world))]
    if bs <= 0 or n_heads <= 0 or world <= 0 or n_tok <= 0:
        raise ValueError("bad partition request bs=%r heads=%r n_tok=%r world=%r" % (bs, n_heads, n_tok, world))
    out = []
    for b in range(bs):
        r0, r1 = shard_range(world, b, bs)
        hs, g = _grid_shape(r1 - r0, n_heads, n_tok, lane_heads)
        if hs > n_heads:
            raise ValueError("%d ranks for one batch item but only %d heads" % (r1 - r0, n_heads))
        for j in range(hs):
            h0, h1 = shard_range(n_heads, j, hs)
            base = r0 + j * g * g
            for ti in range(g):
                for si in range(g):
                    t0, t1 = shard_range(n_tok, ti, g)
                    s0, s1 = shard_range(n_tok, si, g)
                    out.append(dict(b0=b, b1=b + 1, h0=h0, h1=h1, t0=t0, t1=t1, s0=s0, s1=s1,
                                    row=[base + ti * g + x for x in range(g)],
                                    col=[base + x * g + si for x in range(g)]))
    return out


def _cuda_dense_ops():
    import l1attn_cabi as cabi

    class Ops:
        def forward(self, q, k, out):
            return cabi.dense_fwd(q, k, out=out)

        def backward(self, d_attn, q, k, out, scratch):
            return cabi.dense_bwd(d_attn, q, k, out=out, scratch=scratch if scratch is not None else "auto")

        def scratch(self, q):
            import torch as _t
            n = cabi.lib().l1attn_dense_bwd_scratch_bytes(q.shape[0], q.shape[1], q.shape[2], q.shape[3], cabi._tdt(q))
            return _t.empty(max(int(n), 1), dtype=_t.uint8, device=q.device)
    return Ops()


_GROUPS = {}  # process groups by rank tuple: created once per process, whatever number of plans is built


class DenseGridShard:
    """L1Attn forward + backward of ONE global problem [bs, n_tok, n_heads, width] over `world` ranks.

    Every rank runs the single-GPU operator on a square block: queries q[b, t0:t1, h0:h1], keys k[b, s0:s1, h0:h1]
    -> scores attn[b, s0:s1, t0:t1, h0:h1], which stay on the rank.  In the backward the rank's d_q covers its
    query rows but only the keys of its block, and its d_k its key rows but only its queries: ONE all-reduce of
    d_q over the ranks of the same query block and ONE of d_k over those of the same key block complete them
    (none when a rank holds whole batch items).  All ranks must construct this object at the same point: it
    creates the process groups it needs (once per process and set of ranks).  No kernel reads another GPU's memory; the sums go through torch.distributed.

    `ops` is the compute backend (default: this library; the CPU tests of the partition logic pass a stand-in)."""

    def __init__(self, bs, n_tok, n_heads, rank, world, ops=None, lane_heads=8):
        self.part = dense_grid_partition(bs, n_heads, n_tok, world, lane_heads)
        self.me = self.part[rank]
        self.rank, self.world = rank, world
        self.ops = ops if ops is not None else _cuda_dense_ops()
        self.row_group = self.col_group = None
        # every rank creates every group, in the same order (new_group is collective over the whole job)
        if world > 1 and dist.is_available() and dist.is_initialized():
            for p in self.part:
                for key in (tuple(p["row"]), tuple(p["col"])):
                    if len(key) > 1 and key not in _GROUPS:
                        _GROUPS[key] = dist.new_group(list(key))
            self.row_group = _GROUPS.get(tuple(self.me["row"]))
            self.col_group = _GROUPS.get(tuple(self.me["col"]))
        self._scratch = None

    def local_inputs(self, q, k):
        """The rank's contiguous blocks of the global q and k."""
        m = self.me
        return (q[m["b0"]:m["b1"], m["t0"]:m["t1"], m["h0"]:m["h1"]].contiguous(),
                k[m["b0"]:m["b1"], m["s0"]:m["s1"], m["h0"]:m["h1"]].contiguous())

    def local_scores(self, attn):
        """The rank's block of a global [bs, n_tok, n_tok, n_heads] tensor in the layout of the scores."""
        m = self.me
        return attn[m["b0"]:m["b1"], m["s0"]:m["s1"], m["t0"]:m["t1"], m["h0"]:m["h1"]].contiguous()

    def forward(self, q_loc, k_loc, out=None):
        return self.ops.forward(q_loc, k_loc, out)

    def backward(self, d_attn_loc, q_loc, k_loc, out=None):
        """Returns (d_q of the rank's query rows, d_k of its key rows), complete after the two all-reduces."""
        if self._scratch is None or self._scratch_for != tuple(q_loc.shape):
            self._scratch = self.ops.scratch(q_loc)
            self._scratch_for = tuple(q_loc.shape)
        d_q, d_k = self.ops.backward(d_attn_loc, q_loc, k_loc, out, self._scratch)
        if self.row_group is not None:
            dist.all_reduce(d_q, group=self.row_group)
        if self.col_group is not None:
            dist.all_reduce(d_k, group=self.col_group)
        return d_q, d_k

    def describe(self):
        m = self.me
        return ("rank %d: batch %d..%d, heads %d..%d, query rows %d..%d, key rows %d..%d"
                % (self.rank, m["b0"], m["b1"], m["h0"], m["h1"], m["t0"], m["t1"], m["s0"], m["s1"]))

    def collective_note(self):
        m = self.me
        if len(m["row"]) == 1 and len(m["col"]) == 1:
            return None
        return ("all_reduce(SUM) of d_q over ranks %s and of d_k over ranks %s" % (m["row"], m["col"]))


# ------------------------------------------------------------------ sparse: batch items or dst-token ranges

def _cuda_sparse_ops(device):
    """The library's sparse forward/backward behind the (coo -> index) object SparseShard needs."""
    import l1attn_cabi as cabi

    class Ops:
        def index(self, coo, n_tok, dst_mxlen):
            ix = cabi.SparseIndex(coo.to(device), n_tok, dst_mxlen)
            ix.check()
            return ix

        def forward(self, v, q, k, ix, usm, out):
            return cabi.sparse_fwd(v, q, k, ix, usm, out=out)

        def backward(self, dvo, v, q, k, ix, attn, usm, out, scratch):
            return cabi.sparse_bwd(dvo, v, q, k, ix, attn, usm, out=out, scratch=scratch)

        def expand(self, co):
            coo, dm, _ = cabi.expand_coo_host(co.cpu().numpy())
            return torch.from_numpy(coo), dm
    return Ops()


class SparseShard:
    """L1AttnSparse forward + backward over `world` ranks.

    mode "batch"  (bs >= world): rank r owns batch items shard_range(bs, r, world); nothing is exchanged.
    mode "head"   (bs <  world, and no more ranks per item than heads): the operator is independent per (batch item,
                  head) too, so the ranks of one item split its heads (dense_partition); every rank works on
                  contiguous [B_loc, n, H_loc, W] copies of q, k, v with the full graph; nothing is exchanged.
    mode "dst"    (what is left, or on request): every rank keeps q, k, v (replicated) and owns the dst tokens
                  shard_range(n_tok, r, world): it runs the operator on the sub-list of edges whose dst it
                  owns.  All edges of a dst stay together and keep their order, so their softmax slots are
                  those of the full list; vo, attn and d_q rows of the owned tokens are complete (other rows
                  are zero).  d_k and d_v scatter to arbitrary src tokens, so each rank holds partial sums:
                  they are written into ONE flat buffer and summed with ONE all-reduce.  That all-reduce moves
                  as many bytes as d_k and d_v have, whatever the rank count, so this mode pays only where the
                  kernels take much longer than it.

    `mode` = "auto" picks the first of these that applies.  `n_heads` is needed for "head" (without it "auto" skips
    that mode).  `ops` is the compute backend (default: this library on `device`; there is no CPU implementation --
    the CPU tests of the partition logic pass a stand-in)."""

    def __init__(self, co, bs, n_tok, rank, world, device="cuda", ops=None, n_heads=None, mode="auto"):
        self.bs, self.n_tok, self.rank, self.world, self.device = bs, n_tok, rank, world, device
        self.ops = ops if ops is not None else _cuda_sparse_ops(device)
        co = torch.as_tensor(co)
        if mode not in ("auto", "batch", "head", "dst"):
            raise ValueError("unknown mode %r" % (mode,))
        if mode == "auto":
            ranks_per_item = -(-world // max(bs, 1))
            mode = "batch" if bs >= world else ("head" if n_heads is not None and ranks_per_item <= n_heads else "dst")
        if mode == "batch" and bs < world:
            raise ValueError("batch mode needs at least as many batch items (%d) as ranks (%d)" % (bs, world))
        self.mode = mode
        self.h0, self.h1 = 0, n_heads
        self.d0, self.d1 = 0, n_tok
        mine = co
        if mode == "batch":
            self.b0, self.b1 = shard_range(bs, rank, world)
        elif mode == "head":
            if n_heads is None:
                raise ValueError("head mode needs n_heads")
            self.b0, self.b1, self.h0, self.h1 = dense_partition(bs, n_heads, world)[rank]
        else:
            self.b0, self.b1 = 0, bs
            self.d0, self.d1 = shard_range(n_tok, rank, world)
            mine = co[(co[:, 0] >= self.d0) & (co[:, 0] < self.d1)]
        self.n_edges_local, self.n_edges = int(mine.shape[0]), int(co.shape[0])
        coo, self.dst_mxlen = self.ops.expand(mine)
        self.index = self.ops.index(coo, n_tok, self.dst_mxlen)
        self._buf = None

    def describe(self):
        if self.mode == "batch":
            return "batch items %d..%d of %d on rank %d, full graph, no collective" % (self.b0, self.b1, self.bs, self.rank)
        if self.mode == "head":
            return ("batch items %d..%d, heads %d..%d on rank %d, full graph, no collective"
                    % (self.b0, self.b1, self.h0, self.h1, self.rank))
        return ("dst tokens %d..%d of %d on rank %d (%d of %d edges), q, k, v replicated"
                % (self.d0, self.d1, self.n_tok, self.rank, self.n_edges_local, self.n_edges))

    def collective_note(self):
        if self.mode != "dst" or self._buf is None:
            return None
        return "one all_reduce(SUM) of d_k and d_v in one buffer: %d bytes per rank" % (self._buf.numel() * self._buf.element_size())

    def forward_backward(self, v, q, k, dvo, use_softmax=True):
        """Returns (vo, d_v, d_q, d_k).  batch mode: the rank's batch slice of each; head mode: its (batch, head)
        slab.  dst mode: vo and d_q hold the owned dst rows (zero elsewhere); d_v and d_k are complete on every
        rank after the all-reduce."""
        sl = slice(self.b0, self.b1)
        if self.mode == "head":
            v, q, k, dvo = (t[sl, :, self.h0:self.h1].contiguous() for t in (v, q, k, dvo))
        else:
            v, q, k, dvo = v[sl], q[sl], k[sl], dvo[sl]
        bs, n, h, w = q.shape
        wv = v.shape[3]
        if self._buf is None or self._buf.dtype != q.dtype or self._buf.numel() != k.numel() + v.numel():
            self._buf = torch.empty(k.numel() + v.numel(), dtype=q.dtype, device=q.device)
            self._vo = torch.empty_like(v)
            self._attn = torch.empty((bs, n, self.dst_mxlen, h), dtype=q.dtype, device=q.device)
            self._scratch = torch.empty_like(self._attn)
            self._dq = torch.empty_like(q)
        d_k = self._buf[: k.numel()].view(k.shape)
        d_v = self._buf[k.numel():].view(v.shape)
        vo, attn = self.ops.forward(v, q, k, self.index, use_softmax, (self._vo, self._attn))
        self.ops.backward(dvo, v, q, k, self.index, attn, use_softmax, (d_v, None, self._dq, d_k), self._scratch)
        if self.mode == "dst" and self.world > 1:
            dist.all_reduce(self._buf)
        return vo, d_v, self._dq, d_k
