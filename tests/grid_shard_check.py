"""Run under torch.distributed.run with one rank per GPU (launched by test_modules_gpu.py when the box has the GPUs):
the dense operator over DenseGridShard's square blocks, and the sparse operator over SparseShard's head groups and
dst-token ranges, against the single-GPU operators on the whole problem.
Rank 0 prints "grid-ok" when every rank agrees."""
import os
import sys

import torch
import torch.distributed as dist

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.join(os.path.dirname(HERE), "l1-attention_b200"))


def main():
    import l1attn_cabi as cabi
    import l1attn_shard as sh
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", rank)))
    dev = torch.device("cuda")
    dist.init_process_group("nccl")
    bad = 0
    for shape in [(1, 256, 8, 64), (1, 192, 16, 32), (2, 128, 8, 64)]:
        bs, n, h, w = shape
        gen = torch.Generator(device=dev).manual_seed(11)  # the same global tensors on every rank
        q, k = (torch.randn(shape, generator=gen, device=dev) for _ in range(2))
        g = torch.randn((bs, n, n, h), generator=gen, device=dev)
        k[0, 3] = q[0, 5]  # exact ties that cross block borders when the tokens are split
        k[0, n - 2] = q[0, 1]
        plan = sh.DenseGridShard(bs, n, h, rank, world)
        ql, kl = plan.local_inputs(q, k)
        attn = plan.forward(ql, kl)
        dq, dk = plan.backward(plan.local_scores(g), ql, kl)
        ref = cabi.dense_fwd(q, k)
        rdq, rdk = cabi.dense_bwd(g, q, k)
        m = plan.me
        rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-30))
        errs = (rel(attn, plan.local_scores(ref)),
                rel(dq, rdq[m["b0"]:m["b1"], m["t0"]:m["t1"], m["h0"]:m["h1"]]),
                rel(dk, rdk[m["b0"]:m["b1"], m["s0"]:m["s1"], m["h0"]:m["h1"]]))
        if not (errs[0] == 0.0 and errs[1] < 1e-5 and errs[2] < 1e-5):  # scores: same kernel, same operands; sums: other order
            print("rank %d shape %s: %s  %s" % (rank, shape, errs, plan.describe()), flush=True)
            bad += 1
    # the sparse operator by (batch item, head group) and by dst-token range (one all-reduce of d_k, d_v) against
    # the single-GPU operator on the whole problem
    bs, n, h, w = 1, 300, 8, 32
    gen = torch.Generator().manual_seed(13)
    co = torch.stack([torch.randint(0, n, (2500,), generator=gen), torch.randint(0, n, (2500,), generator=gen)], 1)
    geng = torch.Generator(device=dev).manual_seed(17)
    q, k = (0.5 * torch.randn((bs, n, h, w), generator=geng, device=dev) for _ in range(2))
    v, dvo = (torch.randn((bs, n, h, w), generator=geng, device=dev) for _ in range(2))
    whole = sh.SparseShard(co, bs, n, 0, 1, device=dev, n_heads=h)
    ref = [x.clone() for x in whole.forward_backward(v, q, k, dvo, True)]
    rel = lambda a, b: float((a - b).norm() / b.norm().clamp_min(1e-30))
    for mode in ("head", "dst"):
        plan = sh.SparseShard(co, bs, n, rank, world, device=dev, n_heads=h, mode=mode)
        got = plan.forward_backward(v, q, k, dvo, True)
        if mode == "head":
            sl = (slice(plan.b0, plan.b1), slice(None), slice(plan.h0, plan.h1))
            errs = [rel(g, r[sl]) for g, r in zip(got, ref)]
        else:
            rows = (slice(None), slice(plan.d0, plan.d1))
            errs = [rel(got[0][rows], ref[0][rows]), rel(got[1], ref[1]), rel(got[2][rows], ref[2][rows]), rel(got[3], ref[3])]
        if not all(e < 1e-5 for e in errs):
            print("rank %d sparse %s: %s  %s" % (rank, mode, errs, plan.describe()), flush=True)
            bad += 1
    t = torch.tensor([bad], device=dev)
    dist.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("grid-ok", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if int(t.item()) else 0)


if __name__ == "__main__":
    main()
