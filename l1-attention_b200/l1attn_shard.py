"""Partitioning of the L1-attention operators across the GPUs of one node.

Both operators are independent per batch item (and per head): no reduction crosses items, in the
forward or in the backward.  So the multi-GPU form is one process per GPU, each running the
single-GPU operators on its own slice of the batch, with no collective on the data path; a gather
of the outputs is only needed if one rank wants everything.

  shard_range(n, rank, world)        contiguous, balanced slice [lo, hi) of n items for `rank`
  max_over_ranks(x)                  all-reduce MAX of a python float (for timing: slowest rank)
  gather_batch(t, n_total)           all-gather of batch slices (dim 0) into the full tensor, any rank sizes

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
