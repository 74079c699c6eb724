"""Run under torch.distributed.run with one rank per GPU (launched by test_modules_gpu.py when the box has the GPUs):
the dense operator over DenseGridShard's square blocks against the single-GPU operator on the whole problem.
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
    t = torch.tensor([bad], device=dev)
    dist.all_reduce(t)
    if rank == 0 and int(t.item()) == 0:
        print("grid-ok", flush=True)
    dist.destroy_process_group()
    sys.exit(1 if int(t.item()) else 0)


if __name__ == "__main__":
    main()
